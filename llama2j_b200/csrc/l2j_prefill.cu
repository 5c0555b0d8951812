// Batched prompt processing: the positions of a prompt go through every layer 64 at a time, so a weight byte
// is read from HBM once per 64 tokens instead of once per token, and the dot products run on the tensor cores.
//
// The reference has no such path: its run loop pushes every prompt token through the decode step
// (Run.java:623-637).  What is computed per position is the decode step's arithmetic (Run.java:418-508): the
// same RMSNorm, the same 24-bit fixed-point form of the activations (one power-of-two scale per quantisation
// group, three balanced signed byte limbs), exact integer sums of u8 weights x s8 limbs, (min, scale) of the
// weight group applied in FP32 -- only the order of the FP32 additions over the groups of a row differs from
// the decode kernels, so prompt positions agree with them to rounding, not bit for bit.
//
// Kernels:
//   pf_embed_kernel     rows of the embedding table for the chunk's tokens
//   pf_limbs_kernel     activations -> limbs [3 x 64 rows][K] (the B operand) + per (group, token) unit and sum;
//                       input is RMSNorm(x) * w, the attention output, or SwiGLU(h1, h3)
//   pf_gemm_kernel      C[64 tokens][rows] (+)= W[rows][K] x limbs: TMA (cp.async.bulk.tensor) feeds 128-byte-
//                       swizzled tiles to tcgen05.mma kind::i8 (u8 x s8 -> s32, M 128, N 192, K 32), one
//                       accumulator per quantisation group in tensor memory, double-buffered; four epilogue warps
//                       read it back (tcgen05.ld), scale in FP32 and keep the row sums in registers
//   pf_rope_kv_kernel   RoPE on q and k, rows of the K/V cache (ApplyRope.java:61-92, Run.java:443-455)
//   pf_attention_kernel causal attention of the chunk's queries over the cache, FP32, online softmax

#include "l2j_device.cuh"
#include "l2j_internal.h"

#include <cuda.h>

#include <cfloat>
#include <cmath>
#include <mutex>
#include <vector>

#define PF_DS_WAIT_TIMEOUT 0x1u   // L2J_DS_WAIT_TIMEOUT of the public header

namespace l2j {

namespace {

constexpr int kT = kPrefillTokens;          // tokens per chunk
constexpr int kN = 3 * kT;                  // columns of the B operand: three limbs per token
constexpr int kTileM = 128;                 // weight rows per tile
constexpr int kGemmThreads = 256;
constexpr int kStages = 2;                  // one stage = one quantisation group (K = 256) of A and B
constexpr int kABytes = kTileM * 128;       // one 128-byte-wide half of the A stage
constexpr int kBBytes = kN * 128;
constexpr int kStageBytes = 2 * kABytes + 2 * kBBytes;
constexpr int kAccCols = 256;               // column distance of the two accumulators in tensor memory
constexpr int kTmemCols = 512;

// ---- tcgen05 / TMA wrappers ----------------------------------------------------------------------------------

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
                 : "memory");
}

__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar, uint64_t policy)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "l"(policy)
        : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t cols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(cols) : "memory");
}

__device__ __forceinline__ void tmem_relinquish()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

__device__ __forceinline__ void tc_fence_before()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem] x B[smem], u8 x s8 -> s32
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// The barrier gets one arrival when every tcgen05 operation this thread has issued so far is complete.
__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_wait()
{
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, 128-byte swizzled (what the TMA
// writes with CU_TENSOR_MAP_SWIZZLE_128B): groups of 8 rows are 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr)
{
    uint64_t d = (uint64_t)((addr >> 4) & 0x3fffu);
    d |= (uint64_t)1 << 16;                 // leading byte offset (not used by swizzled K-major layouts)
    d |= (uint64_t)(1024 >> 4) << 32;       // stride byte offset
    d |= (uint64_t)1 << 46;                 // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                 // 128-byte swizzle
    return d;
}

// c s32, a u8, b s8, both K-major, N 192, M 128
constexpr uint32_t kIdesc = (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t)(kN >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);

// Bounded wait that also ends when another role of the block has given up.
__device__ __forceinline__ bool pf_wait(uint32_t bar, uint32_t parity, volatile int *give_up, long long limit)
{
    if (mbar_try_wait(bar, parity))
        return true;
    const long long c0 = sm_clock();
    for (;;) {
        if (mbar_try_wait(bar, parity))
            return true;
        if (*give_up != 0 || sm_clock() - c0 > limit) {
            *give_up = 1;
            return false;
        }
    }
}

__device__ __forceinline__ int dp4a_ones(uint32_t limbs, int acc)
{
    int r;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(r) : "r"(0x01010101u), "r"(limbs), "r"(acc));
    return r;
}

}  // namespace

// ---------------------------------------------------------------------------------------------------------------
// GEMM
// ---------------------------------------------------------------------------------------------------------------

struct PfGemmSeg {
    const float2 *hdr;   // (min, scale) of group g of row r at hdr[r * groups + g]
    int rows;            // multiple of 128
    int col0;            // first output column of the segment
};

struct PfGemmParams {
    PfGemmSeg seg[3];
    int nseg;
    int groups;          // K / 256
    const float2 *ux;    // [groups][64]: (value of one unit of the integer sums, sum of the fixed-point activations)
    float *out;          // [64][ldc]
    int ldc;
    int accumulate;      // 1: out += result (the residual stream)
    int nvalid;          // tokens of the chunk that exist
    int timeout_us;
    unsigned int *status;
};

__global__ void __launch_bounds__(kGemmThreads, 1)
pf_gemm_kernel(const __grid_constant__ CUtensorMap map_a0, const __grid_constant__ CUtensorMap map_a1,
               const __grid_constant__ CUtensorMap map_a2, const __grid_constant__ CUtensorMap map_b, const PfGemmParams p)
{
    extern __shared__ unsigned char pf_smem_raw[];
    __shared__ __align__(8) unsigned long long s_bar[2 * kStages + 4 + 1];
    __shared__ uint32_t s_tmem;
    __shared__ int s_give_up;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t base = (smem_u32(pf_smem_raw) + 1023u) & ~1023u;            // swizzled tiles want 1024-byte alignment
    unsigned char *gen = pf_smem_raw + (base - smem_u32(pf_smem_raw));
    float2 *s_ux = reinterpret_cast<float2 *>(gen + kStages * kStageBytes);
    const uint32_t bar_full = smem_u32(&s_bar[0]), bar_empty = smem_u32(&s_bar[kStages]);
    const uint32_t bar_acc_full = smem_u32(&s_bar[2 * kStages]), bar_acc_empty = smem_u32(&s_bar[2 * kStages + 2]);
    const uint32_t bar_fin = smem_u32(&s_bar[2 * kStages + 4]);
    const long long limit = 2000ll * (long long)p.timeout_us;

    int ntiles = 0;
    for (int s = 0; s < p.nseg; ++s)
        ntiles += p.seg[s].rows / kTileM;
    const int G = p.groups;

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_acc_full + 8 * b, 1);
            mbar_init(bar_acc_empty + 8 * b, 4);
        }
        mbar_init(bar_fin, 1);
        mbar_fence_init();
        s_give_up = 0;
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&s_tmem), kTmemCols);
        tmem_relinquish();
    }
    for (int i = tid; i < G * kT; i += kGemmThreads)
        s_ux[i] = p.ux[i];
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    volatile int *give_up = &s_give_up;

    if (warp == 0) {
        // ---- producer: one lane feeds the stages
        if (lane == 0) {
            const uint64_t pol = policy_evict_first();
            long it = 0;
            for (int tile = blockIdx.x; tile < ntiles && !*give_up; tile += gridDim.x) {
                int sg = 0, m0 = tile * kTileM;
                while (m0 >= p.seg[sg].rows) {
                    m0 -= p.seg[sg].rows;
                    ++sg;
                }
                const CUtensorMap *ma = sg == 0 ? &map_a0 : (sg == 1 ? &map_a1 : &map_a2);
                for (int g = 0; g < G; ++g, ++it) {
                    const int s = (int)(it % kStages);
                    const uint32_t ph = (uint32_t)((it / kStages) & 1);
                    if (!pf_wait(bar_empty + 8 * s, ph ^ 1u, give_up, limit))
                        break;
                    const uint32_t st = base + (uint32_t)s * kStageBytes;
                    mbar_arrive_expect_tx(bar_full + 8 * s, kStageBytes);
                    tma_load_2d_hint(st, ma, g * 256, m0, bar_full + 8 * s, pol);
                    tma_load_2d_hint(st + kABytes, ma, g * 256 + 128, m0, bar_full + 8 * s, pol);
                    tma_load_2d(st + 2 * kABytes, &map_b, g * 256, 0, bar_full + 8 * s);
                    tma_load_2d(st + 2 * kABytes + kBBytes, &map_b, g * 256 + 128, 0, bar_full + 8 * s);
                }
            }
            if (*give_up) {
                // copies that nobody consumed must land before the block's shared memory goes away
                for (int s = 0; s < kStages; ++s)
                    for (uint32_t ph = 0; ph < 2; ++ph) {
                        const long long c0 = sm_clock();
                        while (!mbar_try_wait(bar_full + 8 * s, ph) && sm_clock() - c0 < limit) {
                        }
                    }
            }
        }
    } else if (warp == 1) {
        // ---- tensor-core issue: one lane
        if (lane == 0) {
            long it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
                for (int g = 0; g < G; ++g, ++it) {
                    const int s = (int)(it % kStages), b = (int)(it & 1);
                    const uint32_t ph = (uint32_t)((it / kStages) & 1), pha = (uint32_t)((it >> 1) & 1);
                    if (!pf_wait(bar_acc_empty + 8 * b, pha ^ 1u, give_up, limit) || !pf_wait(bar_full + 8 * s, ph, give_up, limit)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t st = base + (uint32_t)s * kStageBytes;
                    const uint32_t d = tmem + (uint32_t)b * kAccCols;
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk) {
                        const uint32_t a_addr = st + (uint32_t)(kk >> 2) * kABytes + (uint32_t)(kk & 3) * 32u;
                        const uint32_t b_addr = st + 2 * kABytes + (uint32_t)(kk >> 2) * kBBytes + (uint32_t)(kk & 3) * 32u;
                        umma_i8(d, smem_desc_sw128(a_addr), smem_desc_sw128(b_addr), kIdesc, kk > 0 ? 1u : 0u);
                    }
                    umma_commit(bar_empty + 8 * s);        // the stage may be refilled when these have read it
                    umma_commit(bar_acc_full + 8 * b);     // and the group's sums are complete
                }
            }
            if (!ok) {
                umma_commit(bar_fin);
                const long long c0 = sm_clock();
                while (!mbar_try_wait(bar_fin, 0) && sm_clock() - c0 < limit) {
                }
            }
        }
    } else if (warp >= 4) {
        // ---- epilogue: thread = one row of the tile, 64 token sums in registers
        const int q = warp & 3;                               // the quarter of tensor memory this warp may read
        const uint32_t trow = tmem + ((uint32_t)(q * 32) << 16);
        long it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
            int sg = 0, m0 = tile * kTileM;
            while (m0 >= p.seg[sg].rows) {
                m0 -= p.seg[sg].rows;
                ++sg;
            }
            const int row = m0 + q * 32 + lane;
            const float2 *hrow = p.seg[sg].hdr + (size_t)row * G;
            float acc[kT];
#pragma unroll
            for (int t = 0; t < kT; ++t)
                acc[t] = 0.f;
            float2 ms = hrow[0];
            for (int g = 0; g < G; ++g, ++it) {
                const int b = (int)(it & 1);
                const uint32_t pha = (uint32_t)((it >> 1) & 1);
                const float2 ms_next = hrow[g + 1 < G ? g + 1 : g];
                if (!pf_wait(bar_acc_full + 8 * b, pha, give_up, limit)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t tacc = trow + (uint32_t)b * kAccCols;
                const float2 *ux = s_ux + g * kT;
#pragma unroll
                for (int t0 = 0; t0 < kT; t0 += 16) {
                    uint32_t s0[16], s1[16], s2[16];
                    tmem_ld16(tacc + t0, s0);
                    tmem_ld16(tacc + kT + t0, s1);
                    tmem_ld16(tacc + 2 * kT + t0, s2);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float dsum = fmaf((float)(int)s2[j], 65536.0f, fmaf((float)(int)s1[j], 256.0f, (float)(int)s0[j]));
                        const float2 u = ux[t0 + j];
                        acc[t0 + j] += fmaf(ms.y, dsum, ms.x * u.y) * u.x;
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(bar_acc_empty + 8 * b);
                ms = ms_next;
            }
            if (ok) {
                float *o = p.out + p.seg[sg].col0 + row;
                if (p.accumulate) {
#pragma unroll
                    for (int t = 0; t < kT; ++t)
                        if (t < p.nvalid)
                            o[(size_t)t * p.ldc] = __fadd_rn(o[(size_t)t * p.ldc], acc[t]);
                } else {
#pragma unroll
                    for (int t = 0; t < kT; ++t)
                        if (t < p.nvalid)
                            o[(size_t)t * p.ldc] = acc[t];
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1)
        tmem_dealloc(tmem, kTmemCols);
    if (tid == 0 && s_give_up)
        atomicOr(p.status, PF_DS_WAIT_TIMEOUT);
}

// ---------------------------------------------------------------------------------------------------------------
// activations -> limbs
// ---------------------------------------------------------------------------------------------------------------

enum { PF_IN_NORM = 0, PF_IN_PLAIN = 1, PF_IN_SWIGLU = 2 };

struct PfLimbParams {
    const float *a;        // [64][lda]: x (NORM), the vector itself (PLAIN), h1 (SWIGLU)
    const float *b;        // NORM: RMSNorm weights [n]; SWIGLU: h3 [64][lda]
    int lda;
    int n;                 // elements per token (multiple of 256)
    int nvalid;
    int8_t *limbs;         // [3 * 64][n]
    float2 *ux;            // [n / 256][64]
};

template <int MODE>
__global__ void __launch_bounds__(256) pf_limbs_kernel(const PfLimbParams p)
{
    __shared__ float s_inv[64];     // value of one fixed-point unit per group (up to 16384 elements per row)
    __shared__ float s_xs[64];
    __shared__ float s_ssq[8];
    const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = p.n >> 8;
    const bool live = t < p.nvalid;
    float ssq = 0.f;
    for (int gi = warp; gi < G; gi += 8) {
        float v[8];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int e = gi * 256 + h * 128 + lane * 4;
            float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
            if (live)
                x = *reinterpret_cast<const float4 *>(p.a + (size_t)t * p.lda + e);
            if (MODE == PF_IN_NORM) {
                const float4 w = *reinterpret_cast<const float4 *>(p.b + e);
                ssq = fmaf(x.x, x.x, ssq); ssq = fmaf(x.y, x.y, ssq); ssq = fmaf(x.z, x.z, ssq); ssq = fmaf(x.w, x.w, ssq);
                x.x = __fmul_rn(w.x, x.x); x.y = __fmul_rn(w.y, x.y); x.z = __fmul_rn(w.z, x.z); x.w = __fmul_rn(w.w, x.w);
            } else if (MODE == PF_IN_SWIGLU) {
                float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
                if (live)
                    y = *reinterpret_cast<const float4 *>(p.b + (size_t)t * p.lda + e);
                // Silu.java:122-132 order: (value * sigmoid) * hb2
                x.x = __fmul_rn(__fmul_rn(x.x, sigmoid_accurate(x.x)), y.x);
                x.y = __fmul_rn(__fmul_rn(x.y, sigmoid_accurate(x.y)), y.y);
                x.z = __fmul_rn(__fmul_rn(x.z, sigmoid_accurate(x.z)), y.z);
                x.w = __fmul_rn(__fmul_rn(x.w, sigmoid_accurate(x.w)), y.w);
            }
            v[4 * h] = x.x; v[4 * h + 1] = x.y; v[4 * h + 2] = x.z; v[4 * h + 3] = x.w;
        }
        float amax = 0.f;
#pragma unroll
        for (int q = 0; q < 8; ++q)
            amax = fmaxf(amax, fabsf(v[q]));
        amax = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(amax)));
        // 24-bit fixed point: one power-of-two scale per group, |x * f| <= 2^22 (the decode kernels' rule)
        int ex = (int)((__float_as_uint(amax) >> 23) & 0xffu) - 126;
        if (!(amax > 0.f) || !(amax < 3.0e38f))
            ex = 0;
        ex = max(-90, min(126, ex));
        const float f = __int_as_float((127 + 22 - ex) << 23);
        uint32_t z[8];
#pragma unroll
        for (int q = 0; q < 8; ++q)
            z[q] = ((uint32_t)__float2int_rn(v[q] * f) + 0x00008080u) ^ 0x00008080u;
        int s0 = 0, s1 = 0, s2 = 0;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t t0 = __byte_perm(z[4 * h], z[4 * h + 1], 0x5140);
            const uint32_t t2 = __byte_perm(z[4 * h + 2], z[4 * h + 3], 0x5140);
            const uint32_t t1 = __byte_perm(z[4 * h], z[4 * h + 1], 0x0062);
            const uint32_t t3 = __byte_perm(z[4 * h + 2], z[4 * h + 3], 0x0062);
            const uint32_t l0 = __byte_perm(t0, t2, 0x5410), l1 = __byte_perm(t0, t2, 0x7632), l2 = __byte_perm(t1, t3, 0x5410);
            const size_t e = (size_t)gi * 256 + h * 128 + lane * 4;
            *reinterpret_cast<uint32_t *>(p.limbs + ((size_t)(0 * kT + t)) * p.n + e) = l0;
            *reinterpret_cast<uint32_t *>(p.limbs + ((size_t)(1 * kT + t)) * p.n + e) = l1;
            *reinterpret_cast<uint32_t *>(p.limbs + ((size_t)(2 * kT + t)) * p.n + e) = l2;
            s0 = dp4a_ones(l0, s0);
            s1 = dp4a_ones(l1, s1);
            s2 = dp4a_ones(l2, s2);
        }
        s0 = __reduce_add_sync(0xffffffffu, s0);
        s1 = __reduce_add_sync(0xffffffffu, s1);
        s2 = __reduce_add_sync(0xffffffffu, s2);
        if (lane == 0) {
            s_inv[gi] = __int_as_float((127 + ex - 22) << 23);
            s_xs[gi] = fmaf((float)s2, 65536.0f, fmaf((float)s1, 256.0f, (float)s0));
        }
    }
    if (MODE == PF_IN_NORM) {
        ssq = warp_sum(ssq);
        if (lane == 0)
            s_ssq[warp] = ssq;
    }
    __syncthreads();
    float ss = 1.0f;
    if (MODE == PF_IN_NORM) {
        float tot = 0.f;
        for (int w = 0; w < 8; ++w)
            tot += s_ssq[w];
        tot = __fdiv_rn(tot, (float)p.n);
        tot = __fadd_rn(tot, 1e-5f);
        ss = __fdiv_rn(1.0f, __fsqrt_rn(tot));   // RootMeanSquare.java:25-35
    }
    for (int gi = tid; gi < G; gi += 256)
        p.ux[(size_t)gi * kT + t] = live ? make_float2(s_inv[gi] * ss, s_xs[gi]) : make_float2(0.f, 0.f);
}

// ---------------------------------------------------------------------------------------------------------------
// embedding rows, RoPE + cache rows
// ---------------------------------------------------------------------------------------------------------------

__global__ void pf_embed_kernel(const int *tokens, int nvalid, const float *emb, int dim, int vocab, float *x)
{
    const int t = blockIdx.x;
    int tok = t < nvalid ? tokens[t] : 0;
    tok = min(max(tok, 0), vocab - 1);
    const float4 *src = reinterpret_cast<const float4 *>(emb + (size_t)tok * dim);
    float4 *dst = reinterpret_cast<float4 *>(x + (size_t)t * dim);
    for (int i = threadIdx.x; i < dim / 4; i += blockDim.x)
        dst[i] = t < nvalid ? src[i] : make_float4(0.f, 0.f, 0.f, 0.f);
}

struct PfRopeParams {
    const float *qkv;      // [64][dim + 2 kv_dim]
    float *q;              // [64][dim]
    float *k_cache, *v_cache;   // layer base, [kv_head][seq][head]
    const float *rope_cos, *rope_sin;   // [seq][head / 2]
    int dim, kv_dim, head, seq_len, pos0, nvalid;
};

__global__ void pf_rope_kv_kernel(const PfRopeParams p)
{
    const int t = blockIdx.x;
    if (t >= p.nvalid)
        return;
    const int pos = p.pos0 + t, half = p.head >> 1;
    const float *row = p.qkv + (size_t)t * (p.dim + 2 * p.kv_dim);
    const float *cs = p.rope_cos + (size_t)pos * half, *sn = p.rope_sin + (size_t)pos * half;
    for (int i = threadIdx.x; i < (p.dim + 2 * p.kv_dim) / 2; i += blockDim.x) {
        const int e = 2 * i;
        const float v0 = row[e], v1 = row[e + 1];
        if (e < p.dim + p.kv_dim) {
            const int r = e < p.dim ? e : e - p.dim;
            const int d = r % p.head;
            const float c = cs[d >> 1], s = sn[d >> 1];
            const float r0 = __fsub_rn(__fmul_rn(v0, c), __fmul_rn(v1, s));   // ApplyRope.java:61-92
            const float r1 = __fadd_rn(__fmul_rn(v0, s), __fmul_rn(v1, c));
            if (e < p.dim) {
                p.q[(size_t)t * p.dim + r] = r0;
                p.q[(size_t)t * p.dim + r + 1] = r1;
            } else {
                float *dst = p.k_cache + ((size_t)(r / p.head) * p.seq_len + pos) * p.head + d;
                dst[0] = r0;
                dst[1] = r1;
            }
        } else {
            const int r = e - p.dim - p.kv_dim;
            float *dst = p.v_cache + ((size_t)(r / p.head) * p.seq_len + pos) * p.head + (r % p.head);
            dst[0] = v0;
            dst[1] = v1;
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// causal attention of the chunk's queries
// ---------------------------------------------------------------------------------------------------------------

struct PfAttnParams {
    const float *q;        // [64][dim] after RoPE
    const float *k_cache, *v_cache;
    float *out;            // [64][dim]
    int dim, head, kv_mul, seq_len, pos0, nvalid;
};

constexpr int kAttnQ = 16;       // queries per block
constexpr int kAttnKeys = 64;    // keys per tile
constexpr int kAttnThreads = 128;

template <int HEAD>
__global__ void __launch_bounds__(kAttnThreads) pf_attention_kernel(const PfAttnParams p)
{
    constexpr int LD = HEAD + 4;             // row pitch in floats: consecutive rows start 4 banks apart
    constexpr int DV = HEAD / 16;            // output elements per thread and query
    extern __shared__ __align__(16) float pf_att_smem[];
    float *sK = pf_att_smem;                 // [64][LD]
    float *sV = sK + kAttnKeys * LD;
    float *sQ = sV + kAttnKeys * LD;         // [16][LD]
    float *sP = sQ + kAttnQ * LD;            // [16][64]

    const int h = blockIdx.x, q0 = blockIdx.y * kAttnQ, tid = threadIdx.x;
    if (q0 >= p.nvalid)
        return;
    const int kvh = h / p.kv_mul;
    const float *kbase = p.k_cache + (size_t)kvh * p.seq_len * HEAD;
    const float *vbase = p.v_cache + (size_t)kvh * p.seq_len * HEAD;
    const int qa = (tid >> 4) * 2;           // this thread's two queries
    const int kb = tid & 15;                 // its keys are kb, kb + 16, kb + 32, kb + 48 of a tile; its outputs DV from kb * DV
    const float root = sqrtf((float)HEAD);   // AttentionLoop: score / sqrt(head_size)

    for (int i = tid; i < kAttnQ * (HEAD / 4); i += kAttnThreads) {
        const int r = i / (HEAD / 4), c = i % (HEAD / 4);
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (q0 + r < p.nvalid)
            v = *reinterpret_cast<const float4 *>(p.q + (size_t)(q0 + r) * p.dim + h * HEAD + c * 4);
        *reinterpret_cast<float4 *>(sQ + r * LD + c * 4) = v;
    }
    float m[2] = {-FLT_MAX, -FLT_MAX}, l[2] = {0.f, 0.f};
    float o[2][DV];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int d = 0; d < DV; ++d)
            o[i][d] = 0.f;

    const int last_q = min(q0 + kAttnQ, p.nvalid) - 1;
    const int nkeys = p.pos0 + last_q + 1;                      // keys 0 .. position of the block's last query
    for (int k0 = 0; k0 < nkeys; k0 += kAttnKeys) {
        __syncthreads();
        for (int i = tid; i < kAttnKeys * (HEAD / 4); i += kAttnThreads) {
            const int r = i / (HEAD / 4), c = i % (HEAD / 4);
            float4 kv = make_float4(0.f, 0.f, 0.f, 0.f), vv = kv;
            if (k0 + r < nkeys) {
                kv = *reinterpret_cast<const float4 *>(kbase + (size_t)(k0 + r) * HEAD + c * 4);
                vv = *reinterpret_cast<const float4 *>(vbase + (size_t)(k0 + r) * HEAD + c * 4);
            }
            *reinterpret_cast<float4 *>(sK + r * LD + c * 4) = kv;
            *reinterpret_cast<float4 *>(sV + r * LD + c * 4) = vv;
        }
        __syncthreads();
        // scores of 2 queries x 4 keys
        float s[2][4];
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
                s[i][j] = 0.f;
#pragma unroll 4
        for (int d = 0; d < HEAD; d += 4) {
            float4 qv[2], kv[4];
#pragma unroll
            for (int i = 0; i < 2; ++i)
                qv[i] = *reinterpret_cast<const float4 *>(sQ + (qa + i) * LD + d);
#pragma unroll
            for (int j = 0; j < 4; ++j)
                kv[j] = *reinterpret_cast<const float4 *>(sK + (kb + 16 * j) * LD + d);
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    s[i][j] = fmaf(qv[i].x, kv[j].x, s[i][j]);
                    s[i][j] = fmaf(qv[i].y, kv[j].y, s[i][j]);
                    s[i][j] = fmaf(qv[i].z, kv[j].z, s[i][j]);
                    s[i][j] = fmaf(qv[i].w, kv[j].w, s[i][j]);
                }
        }
        float alpha[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int qpos = p.pos0 + q0 + qa + i;
            float mx = -FLT_MAX;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int key = k0 + kb + 16 * j;
                s[i][j] = key <= qpos ? __fdiv_rn(s[i][j], root) : -FLT_MAX;
                mx = fmaxf(mx, s[i][j]);
            }
#pragma unroll
            for (int o2 = 1; o2 < 16; o2 <<= 1)
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o2));
            const float mn = fmaxf(m[i], mx);
            alpha[i] = expf(m[i] - mn);
            float sum = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float pv = s[i][j] > -FLT_MAX ? expf(s[i][j] - mn) : 0.f;
                sP[(qa + i) * kAttnKeys + kb + 16 * j] = pv;
                sum += pv;
            }
#pragma unroll
            for (int o2 = 1; o2 < 16; o2 <<= 1)
                sum += __shfl_xor_sync(0xffffffffu, sum, o2);
            l[i] = l[i] * alpha[i] + sum;
            m[i] = mn;
#pragma unroll
            for (int d = 0; d < DV; ++d)
                o[i][d] *= alpha[i];
        }
        __syncthreads();
        const int kmax = min(kAttnKeys, nkeys - k0);
        for (int j = 0; j < kmax; ++j) {
            const float p0 = sP[qa * kAttnKeys + j], p1 = sP[(qa + 1) * kAttnKeys + j];
            const float *vr = sV + j * LD + kb * DV;
#pragma unroll
            for (int d = 0; d < DV; d += 4) {
                const float4 vv = *reinterpret_cast<const float4 *>(vr + d);
                o[0][d] = fmaf(p0, vv.x, o[0][d]); o[0][d + 1] = fmaf(p0, vv.y, o[0][d + 1]);
                o[0][d + 2] = fmaf(p0, vv.z, o[0][d + 2]); o[0][d + 3] = fmaf(p0, vv.w, o[0][d + 3]);
                o[1][d] = fmaf(p1, vv.x, o[1][d]); o[1][d + 1] = fmaf(p1, vv.y, o[1][d + 1]);
                o[1][d + 2] = fmaf(p1, vv.z, o[1][d + 2]); o[1][d + 3] = fmaf(p1, vv.w, o[1][d + 3]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int qi = q0 + qa + i;
        if (qi < p.nvalid) {
            float *dst = p.out + (size_t)qi * p.dim + h * HEAD + kb * DV;
#pragma unroll
            for (int d = 0; d < DV; ++d)
                dst[d] = __fdiv_rn(o[i][d], l[i]);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------------------

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn()
{
    static std::once_flag once;
    static EncodeTiledFn fn = nullptr;
    std::call_once(once, [] {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    });
    return fn;
}

// Byte matrix [rows][k] (row pitch k), tiles of box_rows x 128 bytes, 128-byte swizzled in shared memory.
bool encode_bytes_2d(CUtensorMap *map, const void *base, int rows, int k, int box_rows)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn)
        return false;
    const cuuint64_t gdim[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    const cuuint64_t gstride[1] = {(cuuint64_t)k};
    const cuuint32_t box[2] = {128u, (cuuint32_t)box_rows};
    const cuuint32_t estride[2] = {1u, 1u};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

struct Prefill {
    PrefillModel m;
    int kv_dim = 0, qkv_ld = 0, sms = 0;
    std::vector<CUtensorMap> maps;   // [layer][PF_W_COUNT]
    CUtensorMap map_b_dim, map_b_hidden;
    int *tokens = nullptr;
    float *x = nullptr, *qkv = nullptr, *q = nullptr, *ao = nullptr, *h1 = nullptr, *h3 = nullptr;
    int8_t *limbs = nullptr;
    float2 *ux = nullptr;
    int token_cap = 0;
    size_t gemm_smem_dim = 0, gemm_smem_hidden = 0, attn_smem = 0;
    std::vector<void *> owned;
    unsigned long long launches = 0;
};

bool prefill_supported(const PrefillModel &m)
{
    const int kv_dim = m.n_kv_heads * m.head;
    return m.dim % 256 == 0 && m.hidden % 256 == 0 && kv_dim % kTileM == 0 && m.dim <= 16384 && m.hidden <= 16384 &&
           (m.head == 64 || m.head == 128) && m.n_heads * m.head == m.dim && m.n_layers > 0;
}

void prefill_destroy(Prefill *pf)
{
    if (!pf)
        return;
    for (void *p : pf->owned)
        cudaFree(p);
    delete pf;
}

template <typename T>
static cudaError_t pf_alloc(Prefill *pf, T **out, size_t count)
{
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, count * sizeof(T));
    if (e != cudaSuccess)
        return e;
    pf->owned.push_back(p);
    *out = static_cast<T *>(p);
    return cudaMemset(p, 0, count * sizeof(T));
}

cudaError_t prefill_create(Prefill **out, const PrefillModel &m)
{
    *out = nullptr;
    if (!prefill_supported(m) || (int)m.layers.size() != m.n_layers)
        return cudaErrorInvalidValue;
    Prefill *pf = new Prefill();
    pf->m = m;
    pf->kv_dim = m.n_kv_heads * m.head;
    pf->qkv_ld = m.dim + 2 * pf->kv_dim;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess)
        e = cudaDeviceGetAttribute(&pf->sms, cudaDevAttrMultiProcessorCount, dev);
    const int kmax = m.dim > m.hidden ? m.dim : m.hidden;
    if (e == cudaSuccess) e = pf_alloc(pf, &pf->x, (size_t)kT * m.dim);
    if (e == cudaSuccess) e = pf_alloc(pf, &pf->qkv, (size_t)kT * pf->qkv_ld);
    if (e == cudaSuccess) e = pf_alloc(pf, &pf->q, (size_t)kT * m.dim);
    if (e == cudaSuccess) e = pf_alloc(pf, &pf->ao, (size_t)kT * m.dim);
    if (e == cudaSuccess) e = pf_alloc(pf, &pf->h1, (size_t)kT * m.hidden);
    if (e == cudaSuccess) e = pf_alloc(pf, &pf->h3, (size_t)kT * m.hidden);
    if (e == cudaSuccess) e = pf_alloc(pf, &pf->limbs, (size_t)kN * kmax);
    if (e == cudaSuccess) e = pf_alloc(pf, &pf->ux, (size_t)(kmax / 256) * kT);
    if (e != cudaSuccess) {
        prefill_destroy(pf);
        return e;
    }
    const int rows[PF_W_COUNT] = {m.dim, pf->kv_dim, pf->kv_dim, m.dim, m.hidden, m.hidden, m.dim};
    const int ks[PF_W_COUNT] = {m.dim, m.dim, m.dim, m.dim, m.dim, m.dim, m.hidden};
    pf->maps.resize((size_t)m.n_layers * PF_W_COUNT);
    bool ok = true;
    for (int l = 0; l < m.n_layers && ok; ++l)
        for (int w = 0; w < PF_W_COUNT && ok; ++w)
            ok = encode_bytes_2d(&pf->maps[(size_t)l * PF_W_COUNT + w], m.layers[(size_t)l].w[w], rows[w], ks[w], kTileM);
    ok = ok && encode_bytes_2d(&pf->map_b_dim, pf->limbs, kN, m.dim, kN) && encode_bytes_2d(&pf->map_b_hidden, pf->limbs, kN, m.hidden, kN);
    if (!ok) {
        prefill_destroy(pf);
        return cudaErrorNotSupported;
    }
    pf->gemm_smem_dim = (size_t)kStages * kStageBytes + (size_t)(m.dim / 256) * kT * sizeof(float2) + 1024;
    pf->gemm_smem_hidden = (size_t)kStages * kStageBytes + (size_t)(m.hidden / 256) * kT * sizeof(float2) + 1024;
    const size_t gmax = pf->gemm_smem_dim > pf->gemm_smem_hidden ? pf->gemm_smem_dim : pf->gemm_smem_hidden;
    e = cudaFuncSetAttribute(pf_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gmax);
    const int ld = m.head + 4;
    pf->attn_smem = (size_t)(2 * kAttnKeys * ld + kAttnQ * ld + kAttnQ * kAttnKeys) * sizeof(float);
    if (e == cudaSuccess)
        e = m.head == 128 ? cudaFuncSetAttribute(pf_attention_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pf->attn_smem)
                          : cudaFuncSetAttribute(pf_attention_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pf->attn_smem);
    if (e != cudaSuccess) {
        prefill_destroy(pf);
        return e;
    }
    *out = pf;
    return cudaSuccess;
}

namespace {

cudaError_t launch_gemm(Prefill *pf, cudaStream_t st, int layer, const int *w, int nw, int k, float *out, int ldc, const int *col0,
                        int accumulate, int nvalid)
{
    const PrefillModel &m = pf->m;
    const int rows_of[PF_W_COUNT] = {m.dim, pf->kv_dim, pf->kv_dim, m.dim, m.hidden, m.hidden, m.dim};
    PfGemmParams p{};
    int tiles = 0;
    for (int i = 0; i < nw; ++i) {
        p.seg[i].hdr = m.layers[(size_t)layer].h[w[i]];
        p.seg[i].rows = rows_of[w[i]];
        p.seg[i].col0 = col0[i];
        tiles += rows_of[w[i]] / kTileM;
    }
    p.nseg = nw;
    p.groups = k / 256;
    p.ux = pf->ux;
    p.out = out;
    p.ldc = ldc;
    p.accumulate = accumulate;
    p.nvalid = nvalid;
    p.timeout_us = m.timeout_us;
    p.status = m.status;
    const CUtensorMap *base = &pf->maps[(size_t)layer * PF_W_COUNT];
    const CUtensorMap &a0 = base[w[0]], &a1 = base[w[nw > 1 ? 1 : 0]], &a2 = base[w[nw > 2 ? 2 : 0]];
    const CUtensorMap &b = k == m.dim ? pf->map_b_dim : pf->map_b_hidden;
    const size_t smem = k == m.dim ? pf->gemm_smem_dim : pf->gemm_smem_hidden;
    const int grid = tiles < pf->sms ? tiles : pf->sms;
    pf_gemm_kernel<<<grid, kGemmThreads, smem, st>>>(a0, a1, a2, b, p);
    ++pf->launches;
    return cudaGetLastError();
}

template <int MODE>
cudaError_t launch_limbs(Prefill *pf, cudaStream_t st, const float *a, const float *b, int lda, int n, int nvalid)
{
    PfLimbParams p{};
    p.a = a;
    p.b = b;
    p.lda = lda;
    p.n = n;
    p.nvalid = nvalid;
    p.limbs = pf->limbs;
    p.ux = pf->ux;
    pf_limbs_kernel<MODE><<<kT, 256, 0, st>>>(p);
    ++pf->launches;
    return cudaGetLastError();
}

}  // namespace

#define PF_CK(x)                  \
    do {                          \
        cudaError_t e_ = (x);     \
        if (e_ != cudaSuccess)    \
            return e_;            \
    } while (0)

// Positions pos0 .. pos0 + n - 1 with the input tokens given (host pointer), enqueued on `st`.
cudaError_t prefill_run(Prefill *pf, cudaStream_t st, const int *tokens_host, int n, int pos0)
{
    const PrefillModel &m = pf->m;
    if (n > pf->token_cap) {
        int *t = nullptr;
        PF_CK(cudaMalloc(reinterpret_cast<void **>(&t), sizeof(int) * (size_t)(n + kT)));
        pf->owned.push_back(t);
        pf->tokens = t;
        pf->token_cap = n;
    }
    PF_CK(cudaMemcpyAsync(pf->tokens, tokens_host, sizeof(int) * (size_t)n, cudaMemcpyHostToDevice, st));
    const int dim = m.dim, hidden = m.hidden, kvd = pf->kv_dim;
    const size_t kv_layer = (size_t)m.n_kv_heads * m.seq_len * m.head;
    (void)kv_layer;
    for (int c0 = 0; c0 < n; c0 += kT) {
        const int nv = n - c0 < kT ? n - c0 : kT;
        pf_embed_kernel<<<kT, 256, 0, st>>>(pf->tokens + c0, nv, m.emb, dim, m.vocab, pf->x);
        ++pf->launches;
        PF_CK(cudaGetLastError());
        for (int l = 0; l < m.n_layers; ++l) {
            const PrefillLayerDesc &L = m.layers[(size_t)l];
            PF_CK(launch_limbs<PF_IN_NORM>(pf, st, pf->x, L.rms_att, dim, dim, nv));
            {
                const int w[3] = {PF_WQ, PF_WK, PF_WV}, col0[3] = {0, dim, dim + kvd};
                PF_CK(launch_gemm(pf, st, l, w, 3, dim, pf->qkv, pf->qkv_ld, col0, 0, nv));
            }
            {
                PfRopeParams r{};
                r.qkv = pf->qkv; r.q = pf->q; r.k_cache = L.kc; r.v_cache = L.vc;
                r.rope_cos = m.rope_cos; r.rope_sin = m.rope_sin;
                r.dim = dim; r.kv_dim = kvd; r.head = m.head; r.seq_len = m.seq_len; r.pos0 = pos0 + c0; r.nvalid = nv;
                pf_rope_kv_kernel<<<kT, 256, 0, st>>>(r);
                ++pf->launches;
                PF_CK(cudaGetLastError());
            }
            {
                PfAttnParams a{};
                a.q = pf->q; a.k_cache = L.kc; a.v_cache = L.vc; a.out = pf->ao;
                a.dim = dim; a.head = m.head; a.kv_mul = m.n_heads / m.n_kv_heads; a.seq_len = m.seq_len; a.pos0 = pos0 + c0; a.nvalid = nv;
                const dim3 grid((unsigned)m.n_heads, (unsigned)((nv + kAttnQ - 1) / kAttnQ));
                if (m.head == 128)
                    pf_attention_kernel<128><<<grid, kAttnThreads, pf->attn_smem, st>>>(a);
                else
                    pf_attention_kernel<64><<<grid, kAttnThreads, pf->attn_smem, st>>>(a);
                ++pf->launches;
                PF_CK(cudaGetLastError());
            }
            PF_CK(launch_limbs<PF_IN_PLAIN>(pf, st, pf->ao, nullptr, dim, dim, nv));
            {
                const int w[1] = {PF_WO}, col0[1] = {0};
                PF_CK(launch_gemm(pf, st, l, w, 1, dim, pf->x, dim, col0, 1, nv));
            }
            PF_CK(launch_limbs<PF_IN_NORM>(pf, st, pf->x, L.rms_ffn, dim, dim, nv));
            {
                const int w1[1] = {PF_W1}, w3[1] = {PF_W3}, col0[1] = {0};
                PF_CK(launch_gemm(pf, st, l, w1, 1, dim, pf->h1, hidden, col0, 0, nv));
                PF_CK(launch_gemm(pf, st, l, w3, 1, dim, pf->h3, hidden, col0, 0, nv));
            }
            PF_CK(launch_limbs<PF_IN_SWIGLU>(pf, st, pf->h1, pf->h3, hidden, hidden, nv));
            {
                const int w[1] = {PF_W2}, col0[1] = {0};
                PF_CK(launch_gemm(pf, st, l, w, 1, hidden, pf->x, dim, col0, 1, nv));
            }
        }
    }
    return cudaSuccess;
}

unsigned long long prefill_launches(const Prefill *pf)
{
    return pf ? pf->launches : 0;
}

}  // namespace l2j
