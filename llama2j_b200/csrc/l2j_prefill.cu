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
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <vector>

#define PF_DS_WAIT_TIMEOUT 0x1u   // L2J_DS_WAIT_TIMEOUT of the public header

namespace l2j {

namespace {

constexpr int kT = kPrefillTokens;          // tokens per chunk
constexpr int kN = 3 * kT;                  // columns of the B operand: three limbs per token
constexpr int kTileM = 128;                 // weight rows per tile
constexpr int kGemmThreads = 384;          // producer warp, issue warp, two spare, eight epilogue warps
constexpr int kEpiWarps = 8;                // warps 4..11: quarter of tensor memory = warp % 4, half of the tokens = (warp - 4) / 4
constexpr int kTH = kT / 2;                 // tokens per epilogue thread
constexpr int kStages = 4;                  // ring depth, a power of two known at compile time: the two single-lane issue
                                            // loops are on the critical path (a run-time depth, i.e. a division per stage,
                                            // costs 15 %); one stage = half a quantisation group (K = 128) of A and B
constexpr int kMaxStages = kStages;
constexpr int kABytes = kTileM * 128;       // the A part of a stage: 128 rows of 128 bytes
constexpr int kBBytes = kN * 128;
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kMaxParts = 12;               // parts a row sum (or a query's keys) may be dealt into
constexpr int kWideParts = 3;               // at most this many parts for the wide outputs (QKV, W1/W3): their sums are read back
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

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, "
        "%20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
          "=r"(r[30]), "=r"(r[31])
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
    const float *ssq;    // [nssq][64] partial sums of squares of the input rows (RMSNorm in front), or nullptr
    int nssq;
    int n;               // elements per input row
    float *out;          // [ksplit][64][ldc]
    int ldc;
    int ksplit;          // the groups of a row are dealt to this many blocks; part z goes to out + z * 64 * ldc
    int nvalid;          // tokens of the chunk that exist
    int timeout_us;
    unsigned int *status;
};

__global__ void __launch_bounds__(kGemmThreads, 1)
pf_gemm_kernel(const __grid_constant__ CUtensorMap map_a0, const __grid_constant__ CUtensorMap map_a1,
               const __grid_constant__ CUtensorMap map_a2, const __grid_constant__ CUtensorMap map_b, const PfGemmParams p)
{
    extern __shared__ unsigned char pf_smem_raw[];
    __shared__ __align__(8) unsigned long long s_bar[2 * kMaxStages + 4 + 1];
    __shared__ uint32_t s_tmem;
    __shared__ int s_give_up;
    __shared__ float s_ss[kT];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t base = (smem_u32(pf_smem_raw) + 1023u) & ~1023u;            // swizzled tiles want 1024-byte alignment
    unsigned char *gen = pf_smem_raw + (base - smem_u32(pf_smem_raw));
    float2 *s_ux = reinterpret_cast<float2 *>(gen + (size_t)kStages * kStageBytes);
    const uint32_t bar_full = smem_u32(&s_bar[0]), bar_empty = smem_u32(&s_bar[kMaxStages]);
    const uint32_t bar_acc_full = smem_u32(&s_bar[2 * kMaxStages]), bar_acc_empty = smem_u32(&s_bar[2 * kMaxStages + 2]);
    const uint32_t bar_fin = smem_u32(&s_bar[2 * kMaxStages + 4]);
    const long long limit = 2000ll * (long long)p.timeout_us;

    int ntiles = 0;
    for (int s = 0; s < p.nseg; ++s)
        ntiles += p.seg[s].rows / kTileM;
    ntiles *= p.ksplit;                       // work items: (tile, part of the groups)
    const int G = p.groups;
    const int gper = (G + p.ksplit - 1) / p.ksplit;

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_acc_full + 8 * b, 1);
            mbar_init(bar_acc_empty + 8 * b, kEpiWarps);
        }
        mbar_init(bar_fin, 1);
        mbar_fence_init();
        s_give_up = 0;
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&s_tmem), kTmemCols);
        tmem_relinquish();
    }
    if (tid < kT) {
        // RootMeanSquare.java:25-35: the scalar of the RMSNorm in front multiplies every unit of the token
        float ss = 1.0f;
        if (p.ssq != nullptr) {
            float tot = 0.f;
            for (int y = 0; y < p.nssq; ++y)
                tot += p.ssq[y * kT + tid];
            tot = __fdiv_rn(tot, (float)p.n);
            tot = __fadd_rn(tot, 1e-5f);
            ss = __fdiv_rn(1.0f, __fsqrt_rn(tot));
        }
        s_ss[tid] = ss;
    }
    __syncthreads();
    for (int i = tid; i < G * kT; i += kGemmThreads) {
        const float2 u = p.ux[i];
        s_ux[i] = make_float2(u.x * s_ss[i & (kT - 1)], u.y);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    volatile int *give_up = &s_give_up;

    if (warp == 0) {
        // ---- producer: one lane feeds the ring
        if (lane == 0) {
            const uint64_t pol = policy_evict_first();
            long it = 0;
            for (int tile = blockIdx.x; tile < ntiles && !*give_up; tile += gridDim.x) {
                int sg = 0, m0 = (tile / p.ksplit) * kTileM;
                while (m0 >= p.seg[sg].rows) {
                    m0 -= p.seg[sg].rows;
                    ++sg;
                }
                const CUtensorMap *ma = sg == 0 ? &map_a0 : (sg == 1 ? &map_a1 : &map_a2);
                const int g0 = (tile % p.ksplit) * gper, g1 = min(G, g0 + gper);
                for (int hs = 2 * g0; hs < 2 * g1; ++hs, ++it) {   // half groups
                    const int s = (int)(it % kStages);
                    const uint32_t ph = (uint32_t)((it / kStages) & 1);
                    if (!pf_wait(bar_empty + 8 * s, ph ^ 1u, give_up, limit))
                        break;
                    const uint32_t st = base + (uint32_t)s * kStageBytes;
                    mbar_arrive_expect_tx(bar_full + 8 * s, kStageBytes);
                    tma_load_2d_hint(st, ma, hs * 128, m0, bar_full + 8 * s, pol);
                    tma_load_2d(st + kABytes, &map_b, hs * 128, 0, bar_full + 8 * s);
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
                const int g0 = (tile % p.ksplit) * gper, g1 = min(G, g0 + gper);
                for (int g = g0; g < g1 && ok; ++g, ++it) {
                    const int b = (int)(it & 1);
                    const uint32_t pha = (uint32_t)((it >> 1) & 1);
                    if (!pf_wait(bar_acc_empty + 8 * b, pha ^ 1u, give_up, limit)) {
                        ok = false;
                        break;
                    }
                    const uint32_t d = tmem + (uint32_t)b * kAccCols;
                    for (int half = 0; half < 2; ++half) {
                        const long hit = 2 * it + half;
                        const int s = (int)(hit % kStages);
                        if (!pf_wait(bar_full + 8 * s, (uint32_t)((hit / kStages) & 1), give_up, limit)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after();
                        const uint32_t ta = base + (uint32_t)s * kStageBytes, tb = ta + kABytes;
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk)
                            umma_i8(d, smem_desc_sw128(ta + (uint32_t)kk * 32u), smem_desc_sw128(tb + (uint32_t)kk * 32u), kIdesc,
                                    (half | kk) ? 1u : 0u);
                        umma_commit(bar_empty + 8 * s);        // the stage may be refilled when these have read it
                    }
                    if (ok)
                        umma_commit(bar_acc_full + 8 * b);     // the group's sums are complete
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
        // ---- epilogue: thread = one row of the tile and half of the tokens, 32 sums in registers
        const int q = warp & 3;                               // the quarter of tensor memory this warp may read
        const int th = (warp - 4) >> 2;                       // which half of the tokens
        const uint32_t trow = tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(th * kTH);
        long it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
            int sg = 0, m0 = (tile / p.ksplit) * kTileM;
            while (m0 >= p.seg[sg].rows) {
                m0 -= p.seg[sg].rows;
                ++sg;
            }
            const int z = tile % p.ksplit, g0 = z * gper, g1 = min(G, g0 + gper);
            const int row = m0 + q * 32 + lane;
            const float2 *hrow = p.seg[sg].hdr + (size_t)row * G;
            float acc[kTH];
#pragma unroll
            for (int t = 0; t < kTH; ++t)
                acc[t] = 0.f;
            // The (min, scale) pairs of the row come from HBM, 8 bytes per group and row: they are asked for four
            // groups ahead, or every group would wait one memory latency for its own pair.
            const int glast = g1 > g0 ? g1 - 1 : 0;
            float2 msq[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                msq[j] = hrow[min(g0 + j, glast)];
            for (int gb = g0; gb < g1 && ok; gb += 4) {
                float2 nxt[4];
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    nxt[j] = hrow[min(gb + 4 + j, glast)];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int g = gb + j;
                    if (g >= g1 || !ok)
                        continue;
                    const float2 ms = msq[j];
                    const int b = (int)(it & 1);
                    const uint32_t pha = (uint32_t)((it >> 1) & 1);
                    if (!pf_wait(bar_acc_full + 8 * b, pha, give_up, limit)) {
                        ok = false;
                        continue;
                    }
                    tc_fence_after();
                    const uint32_t tacc = trow + (uint32_t)b * kAccCols;
                    // all of the thread's sums of the group in one round trip, then the accumulator is free again
                    uint32_t s0[kTH], s1[kTH], s2[kTH];
                    static_assert(kTH == 32, "one 32-column load per limb");
                    tmem_ld32(tacc, s0);
                    tmem_ld32(tacc + kT, s1);
                    tmem_ld32(tacc + 2 * kT, s2);
                    tmem_ld_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0)
                        mbar_arrive(bar_acc_empty + 8 * b);
                    const float2 *ux = s_ux + g * kT + th * kTH;
#pragma unroll
                    for (int k = 0; k < kTH; ++k) {
                        const float dsum = fmaf((float)(int)s2[k], 65536.0f, fmaf((float)(int)s1[k], 256.0f, (float)(int)s0[k]));
                        const float2 u = ux[k];
                        acc[k] += fmaf(ms.y, dsum, ms.x * u.y) * u.x;
                    }
                    ++it;
                }
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    msq[j] = nxt[j];
            }
            if (ok) {
                float *o = p.out + (size_t)z * kT * p.ldc + p.seg[sg].col0 + row;
#pragma unroll
                for (int t = 0; t < kTH; ++t)
                    if (th * kTH + t < p.nvalid)
                        o[(size_t)(th * kTH + t) * p.ldc] = acc[t];
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

enum { PF_IN_NORM = 0, PF_IN_ATTN = 1, PF_IN_SWIGLU = 2 };

struct PfLimbParams {
    float *a;              // [64][lda]: x (NORM, updated with the parts), h1 (SWIGLU); ATTN: unused
    const float *b;        // NORM: RMSNorm weights [n]; SWIGLU: h3 [64][lda]
    const float *parts;    // NORM: [nparts][64][lda] partial row sums of the matrix in front, added to x in this order;
                           // ATTN: [nparts][64][heads][head + 2] partial attention outputs (o, m, l) of the key ranges
    int nparts;
    int head;              // ATTN: head size
    int lda;
    int n;                 // elements per token (multiple of 256)
    int nvalid;
    int8_t *limbs;         // [3 * 64][n]
    float2 *ux;            // [n / 256][64]: (value of one fixed-point unit, sum of the fixed-point activations)
    float *ssq;            // NORM: [gridDim.y][64] partial sums of squares of the rows
};

constexpr int kLimbWarps = 4, kLimbThreads = 32 * kLimbWarps;

template <int MODE>
__global__ void __launch_bounds__(kLimbThreads) pf_limbs_kernel(const PfLimbParams p)
{
    // one quantisation group per warp, kLimbWarps groups per block: nothing loops, every load of the block is in
    // flight at once
    __shared__ float s_ssq[kLimbWarps];
    const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = p.n >> 8;
    const bool live = t < p.nvalid;
    float ssq = 0.f;
    const int gi = blockIdx.y * kLimbWarps + warp;
    if (gi < G) {
        float v[8];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int e = gi * 256 + h * 128 + lane * 4;
            float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
            if (live && MODE != PF_IN_ATTN)
                x = *reinterpret_cast<const float4 *>(p.a + (size_t)t * p.lda + e);
            if (MODE == PF_IN_ATTN && live) {
                // the key ranges' partial results of this element's head, merged in a fixed order
                const int hd = e / p.head, d = e - hd * p.head, heads = p.n / p.head, rec = p.head + 2;
                float mx = -FLT_MAX;
                for (int z = 0; z < p.nparts; ++z)
                    mx = fmaxf(mx, p.parts[((size_t)(z * kT + t) * heads + hd) * rec + p.head]);
                float lsum = 0.f;
                for (int z = 0; z < p.nparts; ++z) {
                    const float *r = p.parts + ((size_t)(z * kT + t) * heads + hd) * rec;
                    const float w = expf(r[p.head] - mx);
                    lsum = fmaf(w, r[p.head + 1], lsum);
                    x.x = fmaf(w, r[d], x.x); x.y = fmaf(w, r[d + 1], x.y); x.z = fmaf(w, r[d + 2], x.z); x.w = fmaf(w, r[d + 3], x.w);
                }
                x.x = __fdiv_rn(x.x, lsum); x.y = __fdiv_rn(x.y, lsum); x.z = __fdiv_rn(x.z, lsum); x.w = __fdiv_rn(x.w, lsum);
            }
            if (MODE == PF_IN_NORM && live && p.nparts > 0) {
                for (int z = 0; z < p.nparts; ++z) {
                    const float4 d4 = *reinterpret_cast<const float4 *>(p.parts + ((size_t)z * kT + t) * p.lda + e);
                    x.x = __fadd_rn(x.x, d4.x); x.y = __fadd_rn(x.y, d4.y); x.z = __fadd_rn(x.z, d4.z); x.w = __fadd_rn(x.w, d4.w);
                }
                *reinterpret_cast<float4 *>(p.a + (size_t)t * p.lda + e) = x;   // the residual stream after the matrix in front
            }
            if (MODE == PF_IN_NORM) {
                const float4 w = *reinterpret_cast<const float4 *>(p.b + e);
                ssq = fmaf(x.x, x.x, ssq); ssq = fmaf(x.y, x.y, ssq); ssq = fmaf(x.z, x.z, ssq); ssq = fmaf(x.w, x.w, ssq);
                x.x = __fmul_rn(w.x, x.x); x.y = __fmul_rn(w.y, x.y); x.z = __fmul_rn(w.z, x.z); x.w = __fmul_rn(w.w, x.w);
            } else if (MODE == PF_IN_SWIGLU) {
                float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
                if (live)
                    y = *reinterpret_cast<const float4 *>(p.b + (size_t)t * p.lda + e);
                for (int z = 1; z < p.nparts && live; ++z) {   // split-K parts of h1 and h3, in order
                    const float4 xz = *reinterpret_cast<const float4 *>(p.a + ((size_t)z * kT + t) * p.lda + e);
                    const float4 yz = *reinterpret_cast<const float4 *>(p.b + ((size_t)z * kT + t) * p.lda + e);
                    x.x = __fadd_rn(x.x, xz.x); x.y = __fadd_rn(x.y, xz.y); x.z = __fadd_rn(x.z, xz.z); x.w = __fadd_rn(x.w, xz.w);
                    y.x = __fadd_rn(y.x, yz.x); y.y = __fadd_rn(y.y, yz.y); y.z = __fadd_rn(y.z, yz.z); y.w = __fadd_rn(y.w, yz.w);
                }
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
            const float inv = __int_as_float((127 + ex - 22) << 23);   // value of one fixed-point unit
            const float xs = fmaf((float)s2, 65536.0f, fmaf((float)s1, 256.0f, (float)s0));
            p.ux[(size_t)gi * kT + t] = live ? make_float2(inv, xs) : make_float2(0.f, 0.f);
        }
    }
    if (MODE == PF_IN_NORM) {
        // the row's sum of squares: per block here, summed in block order by the matrix kernel that needs it
        ssq = warp_sum(ssq);
        if (lane == 0)
            s_ssq[warp] = ssq;
        __syncthreads();
        if (tid == 0) {
            float tot = 0.f;
            for (int w = 0; w < kLimbWarps; ++w)
                tot += s_ssq[w];
            p.ssq[(size_t)blockIdx.y * kT + t] = tot;
        }
    }
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
    int nparts;                         // split-K parts of qkv ([nparts][64][dim + 2 kv_dim]), summed here in order
    const int *pos_of, *seq_of;         // concurrent sequences: position and sequence of every token (else pos0 + t, one cache)
    long long seq_stride;               // floats between the caches of two sequences
};

__global__ void pf_rope_kv_kernel(PfRopeParams p)
{
    const int t = blockIdx.x;
    if (t >= p.nvalid)
        return;
    const int pos = p.pos_of ? p.pos_of[t] : p.pos0 + t, half = p.head >> 1;
    if (p.seq_of) {
        p.k_cache += (size_t)p.seq_of[t] * p.seq_stride;
        p.v_cache += (size_t)p.seq_of[t] * p.seq_stride;
    }
    const float *row = p.qkv + (size_t)t * (p.dim + 2 * p.kv_dim);
    const float *cs = p.rope_cos + (size_t)pos * half, *sn = p.rope_sin + (size_t)pos * half;
    const int i = blockIdx.y * blockDim.x + threadIdx.x;      // one pair per thread
    if (i < (p.dim + 2 * p.kv_dim) / 2) {
        const int e = 2 * i;
        float v0 = row[e], v1 = row[e + 1];
        for (int z = 1; z < p.nparts; ++z) {
            const float *rz = row + (size_t)z * kT * (p.dim + 2 * p.kv_dim);
            v0 = __fadd_rn(v0, rz[e]);
            v1 = __fadd_rn(v1, rz[e + 1]);
        }
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
    float *parts;          // [nsplit][64][heads][head + 2]: unnormalised output, running maximum, sum of the key range
    int dim, head, kv_mul, seq_len, pos0, nvalid, nsplit;
};

constexpr int kAttnQ = 32;       // queries per block
constexpr int kAttnKeys = 64;    // keys per tile
constexpr int kAttnThreads = 128;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

__device__ __forceinline__ void cp_async_wait_all()
{
    asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}

// Block = (head, 32 queries, one range of key tiles); thread = 4 queries x 4 keys of a tile for the scores and
// 4 queries x HEAD / 16 elements for the output.  The K and V rows of a tile come into shared memory with
// asynchronous 16-byte copies (no registers, no load-to-store dependency per row); two blocks share an SM.
template <int HEAD>
__global__ void __launch_bounds__(kAttnThreads, 2) pf_attention_kernel(const PfAttnParams p)
{
    constexpr int LD = HEAD + 4;             // row pitch in floats: consecutive rows start 4 banks apart
    constexpr int NV4 = HEAD / 64;           // float4 chunks of the output per thread and query
    extern __shared__ __align__(16) float pf_att_smem[];
    float *sK = pf_att_smem;                 // [64][LD]
    float *sV = sK + kAttnKeys * LD;
    float *sQ = sV + kAttnKeys * LD;         // [32][LD]
    float *sP = sQ + kAttnQ * LD;            // [32][64]

    const int h = blockIdx.x, q0 = blockIdx.y * kAttnQ, z = blockIdx.z, tid = threadIdx.x;
    if (q0 >= p.nvalid)
        return;
    const int kvh = h / p.kv_mul;
    const float *kbase = p.k_cache + (size_t)kvh * p.seq_len * HEAD;
    const float *vbase = p.v_cache + (size_t)kvh * p.seq_len * HEAD;
    const int qa = (tid >> 4) * 4;           // this thread's four queries
    const int kb = tid & 15;                 // its keys are kb, kb + 16, kb + 32, kb + 48 of a tile
    const float root = sqrtf((float)HEAD);   // AttentionLoop: score / sqrt(head_size)

    const int last_q = min(q0 + kAttnQ, p.nvalid) - 1;
    const int nkeys = p.pos0 + last_q + 1;                      // keys 0 .. position of the block's last query
    const int tiles = (nkeys + kAttnKeys - 1) / kAttnKeys;
    const int tper = (tiles + p.nsplit - 1) / p.nsplit;
    const int t_lo = z * tper, t_hi = min(tiles, t_lo + tper);

    for (int i = tid; i < kAttnQ * (HEAD / 4); i += kAttnThreads) {
        const int r = i / (HEAD / 4), c = i % (HEAD / 4);
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (q0 + r < p.nvalid)
            v = *reinterpret_cast<const float4 *>(p.q + (size_t)(q0 + r) * p.dim + h * HEAD + c * 4);
        *reinterpret_cast<float4 *>(sQ + r * LD + c * 4) = v;
    }
    float m[4], l[4];
    float4 o[4][NV4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        m[i] = -FLT_MAX;
        l[i] = 0.f;
#pragma unroll
        for (int c = 0; c < NV4; ++c)
            o[i][c] = make_float4(0.f, 0.f, 0.f, 0.f);
    }

    for (int tile = t_lo; tile < t_hi; ++tile) {
        const int k0 = tile * kAttnKeys;
        __syncthreads();
        for (int i = tid; i < kAttnKeys * (HEAD / 4); i += kAttnThreads) {
            const int r = i / (HEAD / 4), c = i % (HEAD / 4);
            if (k0 + r < nkeys) {
                cp_async16(smem_u32(sK + r * LD + c * 4), kbase + (size_t)(k0 + r) * HEAD + c * 4);
                cp_async16(smem_u32(sV + r * LD + c * 4), vbase + (size_t)(k0 + r) * HEAD + c * 4);
            } else {
                *reinterpret_cast<float4 *>(sK + r * LD + c * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
                *reinterpret_cast<float4 *>(sV + r * LD + c * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        cp_async_wait_all();
        __syncthreads();
        // scores of 4 queries x 4 keys
        float s[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
                s[i][j] = 0.f;
#pragma unroll 2
        for (int d = 0; d < HEAD; d += 4) {
            float4 qv[4], kv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
                qv[i] = *reinterpret_cast<const float4 *>(sQ + (qa + i) * LD + d);
#pragma unroll
            for (int j = 0; j < 4; ++j)
                kv[j] = *reinterpret_cast<const float4 *>(sK + (kb + 16 * j) * LD + d);
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    s[i][j] = fmaf(qv[i].x, kv[j].x, s[i][j]);
                    s[i][j] = fmaf(qv[i].y, kv[j].y, s[i][j]);
                    s[i][j] = fmaf(qv[i].z, kv[j].z, s[i][j]);
                    s[i][j] = fmaf(qv[i].w, kv[j].w, s[i][j]);
                }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
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
            const float alpha = expf(m[i] - mn);
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
            l[i] = l[i] * alpha + sum;
            m[i] = mn;
#pragma unroll
            for (int c = 0; c < NV4; ++c) {
                o[i][c].x *= alpha; o[i][c].y *= alpha; o[i][c].z *= alpha; o[i][c].w *= alpha;
            }
        }
        __syncthreads();
        const int kmax = (min(kAttnKeys, nkeys - k0) + 3) & ~3;   // rows past the last key hold zeros and weigh zero
        for (int j = 0; j < kmax; j += 4) {
            float4 pj[4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
                pj[i] = *reinterpret_cast<const float4 *>(sP + (qa + i) * kAttnKeys + j);
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
#pragma unroll
                for (int c = 0; c < NV4; ++c) {
                    const float4 vv = *reinterpret_cast<const float4 *>(sV + (j + jj) * LD + c * 64 + kb * 4);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float w = jj == 0 ? pj[i].x : (jj == 1 ? pj[i].y : (jj == 2 ? pj[i].z : pj[i].w));
                        o[i][c].x = fmaf(w, vv.x, o[i][c].x); o[i][c].y = fmaf(w, vv.y, o[i][c].y);
                        o[i][c].z = fmaf(w, vv.z, o[i][c].z); o[i][c].w = fmaf(w, vv.w, o[i][c].w);
                    }
                }
            }
        }
    }
    const int heads = p.dim / HEAD;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int qi = q0 + qa + i;
        if (qi < p.nvalid) {
            float *rec = p.parts + ((size_t)(z * kT + qi) * heads + h) * (HEAD + 2);
#pragma unroll
            for (int c = 0; c < NV4; ++c) {   // records are 8-byte aligned (HEAD + 2 floats each)
                *reinterpret_cast<float2 *>(rec + c * 64 + kb * 4) = make_float2(o[i][c].x, o[i][c].y);
                *reinterpret_cast<float2 *>(rec + c * 64 + kb * 4 + 2) = make_float2(o[i][c].z, o[i][c].w);
            }
            if (kb == 0) {
                rec[HEAD] = m[i];
                rec[HEAD + 1] = l[i];
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// concurrent sequences: one decode step of up to 64 (sequence, position) pairs on one sweep over the weights
// ---------------------------------------------------------------------------------------------------------------

struct BdAttnParams {
    const float *q;                     // [64][dim] after RoPE
    const float *k_cache, *v_cache;     // layer base of sequence 0, [kv_head][seq][head]
    long long seq_stride;
    const int *pos_of, *seq_of;
    float *parts;                       // [64][heads][head + 2]: unnormalised output, maximum, sum (one key range)
    int dim, kv_mul, seq_len, nvalid;
};

// Block = (head, token): every token has its own cache and length.  Warp w takes keys 32 (w + 4 i) + lane: the
// lane's dot product with q (shared memory, broadcast), online softmax per warp, then the weighted V rows
// (a row is one coalesced 16-byte load per lane); the four warps merge at the end.
template <int HEAD>
__global__ void __launch_bounds__(128) bd_attention_kernel(const BdAttnParams p)
{
    constexpr int DL = HEAD / 32;       // output elements per lane
    __shared__ __align__(16) float sq[HEAD];
    __shared__ float s_m[4], s_l[4];
    __shared__ __align__(16) float s_o[4][HEAD];
    const int h = blockIdx.x, t = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (t >= p.nvalid)
        return;
    const int pos = p.pos_of[t];
    const size_t cache = (size_t)p.seq_of[t] * p.seq_stride + (size_t)(h / p.kv_mul) * p.seq_len * HEAD;
    const float *kbase = p.k_cache + cache, *vbase = p.v_cache + cache;
    if (tid < HEAD)
        sq[tid] = p.q[(size_t)t * p.dim + h * HEAD + tid];
    __syncthreads();
    const float root = sqrtf((float)HEAD);
    float m = -FLT_MAX, l = 0.f;
    float o[DL];
#pragma unroll
    for (int d = 0; d < DL; ++d)
        o[d] = 0.f;
    for (int k0 = warp * 32; k0 <= pos; k0 += 128) {
        const int key = k0 + lane;
        float sc = -FLT_MAX;
        if (key <= pos) {
            const float4 *kr = reinterpret_cast<const float4 *>(kbase + (size_t)key * HEAD);
            float a = 0.f;
#pragma unroll 8
            for (int d = 0; d < HEAD / 4; ++d) {
                const float4 kv = kr[d];
                const float4 qv = *reinterpret_cast<const float4 *>(sq + 4 * d);
                a = fmaf(qv.x, kv.x, a); a = fmaf(qv.y, kv.y, a); a = fmaf(qv.z, kv.z, a); a = fmaf(qv.w, kv.w, a);
            }
            sc = __fdiv_rn(a, root);
        }
        const float mx = warp_max(sc);
        const float mn = fmaxf(m, mx);
        const float alpha = expf(m - mn);
        const float pv = sc > -FLT_MAX ? expf(sc - mn) : 0.f;
        l = l * alpha + warp_sum(pv);
        m = mn;
#pragma unroll
        for (int d = 0; d < DL; ++d)
            o[d] *= alpha;
        const int kn = min(32, pos + 1 - k0);
        for (int j = 0; j < kn; ++j) {
            const float w = __shfl_sync(0xffffffffu, pv, j);
            const float *vr = vbase + (size_t)(k0 + j) * HEAD + lane * DL;
#pragma unroll
            for (int d = 0; d < DL; ++d)
                o[d] = fmaf(w, vr[d], o[d]);
        }
    }
    if (lane == 0) {
        s_m[warp] = m;
        s_l[warp] = l;
    }
#pragma unroll
    for (int d = 0; d < DL; ++d)
        s_o[warp][lane * DL + d] = o[d];
    __syncthreads();
    const float mt = fmaxf(fmaxf(s_m[0], s_m[1]), fmaxf(s_m[2], s_m[3]));
    float *rec = p.parts + ((size_t)t * (p.dim / HEAD) + h) * (HEAD + 2);
    if (tid < HEAD) {
        float acc = 0.f;
        for (int w = 0; w < 4; ++w)
            acc = fmaf(expf(s_m[w] - mt), s_o[w][tid], acc);
        rec[tid] = acc;
    }
    if (tid == 0) {
        float lt = 0.f;
        for (int w = 0; w < 4; ++w)
            lt = fmaf(expf(s_m[w] - mt), s_l[w], lt);
        rec[HEAD] = mt;
        rec[HEAD + 1] = lt;
    }
}

// x after the last layer (with the partial row sums of its W2), RMSNorm with the final weights
// (RootMeanSquare.java:25-35, WeightNormalizeAndScale.java:71-74): [64][dim] FP32 for the classifier.
__global__ void __launch_bounds__(256) bd_final_norm_kernel(const float *x, const float *parts, int nparts, const float *w, int dim, int nvalid,
                                                            float *out)
{
    __shared__ float s_red[8];
    const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    float ssq = 0.f;
    for (int i = tid; i < dim; i += 256) {
        float v = t < nvalid ? x[(size_t)t * dim + i] : 0.f;
        for (int z = 0; z < nparts && t < nvalid; ++z)
            v = __fadd_rn(v, parts[((size_t)z * kT + t) * dim + i]);
        out[(size_t)t * dim + i] = v;
        ssq = fmaf(v, v, ssq);
    }
    ssq = warp_sum(ssq);
    if (lane == 0)
        s_red[warp] = ssq;
    __syncthreads();
    float tot = 0.f;
    for (int k = 0; k < 8; ++k)
        tot += s_red[k];
    tot = __fdiv_rn(tot, (float)dim);
    tot = __fadd_rn(tot, 1e-5f);
    const float ss = __fdiv_rn(1.0f, __fsqrt_rn(tot));
    for (int i = tid; i < dim; i += 256)
        out[(size_t)t * dim + i] = __fmul_rn(w[i], __fmul_rn(ss, out[(size_t)t * dim + i]));
}

// logits[t][v] = sum_k wcls[v][k] * xn[t][k] for 64 tokens: FP32 on the CUDA cores (the classifier is not
// quantised, TransformerWeights.java:25,41,122), 128 vocabulary rows x 64 tokens per block, K in chunks of 32
// double-buffered with asynchronous copies, 8 rows x 4 tokens per thread.
constexpr int kClsRows = 128, kClsK = 32, kClsLd = kClsK + 4, kClsThreads = 256;
constexpr int kClsStage = (kClsRows + kT) * kClsLd;      // floats per stage

__global__ void __launch_bounds__(kClsThreads) bd_classifier_kernel(const float *wcls, const float *xn, int vocab, int dim, float *logits)
{
    extern __shared__ __align__(16) float cls_smem[];
    const int tid = threadIdx.x, v0 = blockIdx.x * kClsRows;
    const int rg = tid >> 4, tg = tid & 15;          // rows rg + 16 i (i < 8), tokens tg + 16 j (j < 4)
    float acc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
            acc[i][j] = 0.f;
    auto load_stage = [&](int st, int k0) {
        float *sw = cls_smem + st * kClsStage, *sx = sw + kClsRows * kClsLd;
        for (int i = tid; i < (kClsRows + kT) * (kClsK / 4); i += kClsThreads) {
            const int r = i / (kClsK / 4), c = i % (kClsK / 4);
            if (r < kClsRows) {
                const int v = min(v0 + r, vocab - 1);
                cp_async16(smem_u32(sw + r * kClsLd + c * 4), wcls + (size_t)v * dim + k0 + c * 4);
            } else {
                cp_async16(smem_u32(sx + (r - kClsRows) * kClsLd + c * 4), xn + (size_t)(r - kClsRows) * dim + k0 + c * 4);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int nk = dim / kClsK;
    load_stage(0, 0);
    for (int kc = 0; kc < nk; ++kc) {
        if (kc + 1 < nk) {
            load_stage((kc + 1) & 1, (kc + 1) * kClsK);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const float *sw = cls_smem + (kc & 1) * kClsStage, *sx = sw + kClsRows * kClsLd;
#pragma unroll
        for (int k = 0; k < kClsK; k += 4) {
            float4 wv[8], xv[4];
#pragma unroll
            for (int i = 0; i < 8; ++i)
                wv[i] = *reinterpret_cast<const float4 *>(sw + (rg + 16 * i) * kClsLd + k);
#pragma unroll
            for (int j = 0; j < 4; ++j)
                xv[j] = *reinterpret_cast<const float4 *>(sx + (tg + 16 * j) * kClsLd + k);
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = fmaf(wv[i].x, xv[j].x, acc[i][j]);
                    acc[i][j] = fmaf(wv[i].y, xv[j].y, acc[i][j]);
                    acc[i][j] = fmaf(wv[i].z, xv[j].z, acc[i][j]);
                    acc[i][j] = fmaf(wv[i].w, xv[j].w, acc[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int v = v0 + rg + 16 * i;
        if (v < vocab)
#pragma unroll
            for (int j = 0; j < 4; ++j)
                logits[(size_t)(tg + 16 * j) * vocab + v] = acc[i][j];
    }
}

// First maximum of every token's logits (Sampler.java:46-57).
__global__ void __launch_bounds__(256) bd_argmax_kernel(const float *logits, int vocab, int nvalid, int *out)
{
    __shared__ float s_v[8];
    __shared__ int s_i[8];
    const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (t >= nvalid)
        return;
    float bv = -FLT_MAX;
    int bi = 0x7fffffff;
    for (int i = tid; i < vocab; i += 256) {
        const float v = logits[(size_t)t * vocab + i];
        if (v > bv) {
            bv = v;
            bi = i;
        }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) {
            bv = ov;
            bi = oi;
        }
    }
    if (lane == 0) {
        s_v[warp] = bv;
        s_i[warp] = bi;
    }
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < 8; ++w)
            if (s_v[w] > bv || (s_v[w] == bv && s_i[w] < bi)) {
                bv = s_v[w];
                bi = s_i[w];
            }
        out[t] = bi;
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
bool encode_bytes_2d(CUtensorMap *map, const void *base, int rows, int k, int box_rows, bool from_hbm)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn)
        return false;
    const cuuint64_t gdim[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    const cuuint64_t gstride[1] = {(cuuint64_t)k};
    const cuuint32_t box[2] = {128u, (cuuint32_t)box_rows};
    const cuuint32_t estride[2] = {1u, 1u};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, from_hbm ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

struct Prefill {
    PrefillModel m;
    int kv_dim = 0, qkv_ld = 0, sms = 0;
    std::vector<CUtensorMap> maps;   // [layer][PF_W_COUNT]
    CUtensorMap map_b_dim, map_b_hidden;
    int *tokens = nullptr;
    float *x = nullptr, *qkv = nullptr, *q = nullptr, *h13 = nullptr;
    float *parts = nullptr;      // [kMaxParts][64][dim]: partial row sums of Wo / W2, or the attention's key ranges
    int ksplit_o = 1, ksplit_2 = 1, ksplit_qkv = 1, ksplit_13 = 1;
    int8_t *limbs = nullptr;
    float2 *ux = nullptr;
    float *ssq = nullptr;         // [groups / 4][64]
    int token_cap = 0;
    size_t gemm_smem_dim = 0, gemm_smem_hidden = 0, attn_smem = 0;
    std::vector<void *> owned;
    unsigned long long launches = 0;
    // concurrent sequences
    int n_seq = 0, seq_len_b = 0;
    float *bkc = nullptr, *bvc = nullptr;      // [sequence][layer][kv_head][seq_len_b][head]
    int *meta = nullptr;                       // device: tokens[64], positions[64], sequences[64], arg-max[64]
    float *xn = nullptr, *logits = nullptr;    // [64][dim], [64][vocab]
    int *meta_host = nullptr;                  // pinned, 4 x 64
    float *logits_host = nullptr;              // pinned, [64][vocab]
    std::map<int, cudaGraphExec_t> step_graphs; // captured step per entry count
    unsigned long long step_launches = 0;
    bool no_graph = false;
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
    for (auto &g : pf->step_graphs)
        cudaGraphExecDestroy(g.second);
    if (pf->meta_host)
        cudaFreeHost(pf->meta_host);
    if (pf->logits_host)
        cudaFreeHost(pf->logits_host);
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
    if (e == cudaSuccess) e = pf_alloc(pf, &pf->qkv, (size_t)kWideParts * kT * pf->qkv_ld);
    if (e == cudaSuccess) e = pf_alloc(pf, &pf->q, (size_t)kT * m.dim);
    if (e == cudaSuccess) e = pf_alloc(pf, &pf->h13, (size_t)kWideParts * kT * 2 * m.hidden);
    if (e == cudaSuccess) e = pf_alloc(pf, &pf->parts, (size_t)kMaxParts * kT * (m.dim + 2 * m.n_heads));
    if (e == cudaSuccess) e = pf_alloc(pf, &pf->limbs, (size_t)kN * kmax);
    if (e == cudaSuccess) e = pf_alloc(pf, &pf->ux, (size_t)(kmax / 256) * kT);
    if (e == cudaSuccess) e = pf_alloc(pf, &pf->ssq, (size_t)(kmax / 256) * kT);
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
            ok = encode_bytes_2d(&pf->maps[(size_t)l * PF_W_COUNT + w], m.layers[(size_t)l].w[w], rows[w], ks[w], kTileM, true);
    ok = ok && encode_bytes_2d(&pf->map_b_dim, pf->limbs, kN, m.dim, kN, false) &&
         encode_bytes_2d(&pf->map_b_hidden, pf->limbs, kN, m.hidden, kN, false);
    if (!ok) {
        prefill_destroy(pf);
        return cudaErrorNotSupported;
    }
    // ring, unit table (at most 64 groups: 32 KB), alignment slack: below the 227 KB a block may have
    pf->gemm_smem_dim = (size_t)kStages * kStageBytes + (size_t)(m.dim / 256) * kT * sizeof(float2) + 1024;
    pf->gemm_smem_hidden = (size_t)kStages * kStageBytes + (size_t)(m.hidden / 256) * kT * sizeof(float2) + 1024;
    const size_t gmax = pf->gemm_smem_dim > pf->gemm_smem_hidden ? pf->gemm_smem_dim : pf->gemm_smem_hidden;
    e = cudaFuncSetAttribute(pf_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gmax);
    const int ld = m.head + 4;
    pf->attn_smem = (size_t)(2 * kAttnKeys * ld + kAttnQ * ld + kAttnQ * kAttnKeys) * sizeof(float);
    // matrices with few row tiles (Wo, W2: dim / 128) deal the groups of a row to several blocks
    auto split_for = [&](int rows, int groups) {
        int ks = 1;
        while (ks < kMaxParts && (rows / kTileM) * ks * 2 <= pf->sms && groups / (ks * 2) >= 2)
            ks *= 2;
        return ks;
    };
    pf->ksplit_o = split_for(m.dim, m.dim / 256);
    pf->ksplit_2 = split_for(m.dim, m.hidden / 256);
    // the wide matrices have more tiles than SMs or nearly so: the part count that needs the fewest rounds of groups
    auto rounds_split = [&](int tiles, int groups) {
        int best = 1, best_cost = 1 << 30;
        for (int ks = 1; ks <= kWideParts && ks <= groups; ++ks) {
            const int cost = ((tiles * ks + pf->sms - 1) / pf->sms) * ((groups + ks - 1) / ks);
            if (cost < best_cost) {
                best_cost = cost;
                best = ks;
            }
        }
        return best;
    };
    pf->ksplit_qkv = 1;   // measured: three parts for QKV (96 tiles at the 7B shape) gain nothing and cost the RoPE kernel two more reads
    pf->ksplit_13 = rounds_split(2 * m.hidden / kTileM, m.dim / 256);
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
                        int ksplit, int nvalid, bool normed)
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
    p.ksplit = ksplit;
    p.ssq = normed ? pf->ssq : nullptr;
    p.nssq = (k / 256 + kLimbWarps - 1) / kLimbWarps;
    p.n = k;
    p.nvalid = nvalid;
    p.timeout_us = m.timeout_us;
    p.status = m.status;
    const CUtensorMap *base = &pf->maps[(size_t)layer * PF_W_COUNT];
    const CUtensorMap &a0 = base[w[0]], &a1 = base[w[nw > 1 ? 1 : 0]], &a2 = base[w[nw > 2 ? 2 : 0]];
    const CUtensorMap &b = k == m.dim ? pf->map_b_dim : pf->map_b_hidden;
    const size_t smem = k == m.dim ? pf->gemm_smem_dim : pf->gemm_smem_hidden;
    const int grid = tiles * ksplit < pf->sms ? tiles * ksplit : pf->sms;
    pf_gemm_kernel<<<grid, kGemmThreads, smem, st>>>(a0, a1, a2, b, p);
    ++pf->launches;
    return cudaGetLastError();
}

template <int MODE>
cudaError_t launch_limbs(Prefill *pf, cudaStream_t st, float *a, const float *b, const float *parts, int nparts, int lda, int n, int nvalid)
{
    PfLimbParams p{};
    p.a = a;
    p.b = b;
    p.parts = parts;
    p.nparts = nparts;
    p.head = pf->m.head;
    p.lda = lda;
    p.n = n;
    p.nvalid = nvalid;
    p.limbs = pf->limbs;
    p.ux = pf->ux;
    p.ssq = pf->ssq;
    const dim3 grid((unsigned)kT, (unsigned)((n / 256 + kLimbWarps - 1) / kLimbWarps));
    pf_limbs_kernel<MODE><<<grid, kLimbThreads, 0, st>>>(p);
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
        int pending = 0;     // partial row sums in `parts` that the next RMSNorm adds to x
        for (int l = 0; l < m.n_layers; ++l) {
            const PrefillLayerDesc &L = m.layers[(size_t)l];
            PF_CK(launch_limbs<PF_IN_NORM>(pf, st, pf->x, L.rms_att, pf->parts, pending, dim, dim, nv));
            {
                const int w[3] = {PF_WQ, PF_WK, PF_WV}, col0[3] = {0, dim, dim + kvd};
                PF_CK(launch_gemm(pf, st, l, w, 3, dim, pf->qkv, pf->qkv_ld, col0, pf->ksplit_qkv, nv, true));
            }
            {
                PfRopeParams r{};
                r.qkv = pf->qkv; r.q = pf->q; r.k_cache = L.kc; r.v_cache = L.vc;
                r.rope_cos = m.rope_cos; r.rope_sin = m.rope_sin;
                r.dim = dim; r.kv_dim = kvd; r.head = m.head; r.seq_len = m.seq_len; r.pos0 = pos0 + c0; r.nvalid = nv;
                r.nparts = pf->ksplit_qkv;
                const dim3 grid((unsigned)kT, (unsigned)((pf->qkv_ld / 2 + 255) / 256));
                pf_rope_kv_kernel<<<grid, 256, 0, st>>>(r);
                ++pf->launches;
                PF_CK(cudaGetLastError());
            }
            int nsplit = 1;
            {
                const int tiles = (pos0 + c0 + nv + kAttnKeys - 1) / kAttnKeys;
                // key ranges per (head, 32 queries): the count that needs the fewest rounds of key tiles, with two
                // blocks resident per SM (each block pays about half a tile for its set-up and the merge of a part)
                {
                    const int base = m.n_heads * ((nv + kAttnQ - 1) / kAttnQ), places = 2 * pf->sms;
                    float best = 0.f;
                    for (int ns = 1; ns <= kMaxParts && ns <= tiles; ++ns) {
                        const int waves = (base * ns + places - 1) / places;
                        const float cost = (float)waves * ((float)((tiles + ns - 1) / ns) + 0.5f);
                        if (ns == 1 || cost < best) {
                            best = cost;
                            nsplit = ns;
                        }
                    }
                }
                PfAttnParams a{};
                a.q = pf->q; a.k_cache = L.kc; a.v_cache = L.vc; a.parts = pf->parts;
                a.dim = dim; a.head = m.head; a.kv_mul = m.n_heads / m.n_kv_heads; a.seq_len = m.seq_len; a.pos0 = pos0 + c0; a.nvalid = nv;
                a.nsplit = nsplit;
                const dim3 grid((unsigned)m.n_heads, (unsigned)((nv + kAttnQ - 1) / kAttnQ), (unsigned)nsplit);
                if (m.head == 128)
                    pf_attention_kernel<128><<<grid, kAttnThreads, pf->attn_smem, st>>>(a);
                else
                    pf_attention_kernel<64><<<grid, kAttnThreads, pf->attn_smem, st>>>(a);
                ++pf->launches;
                PF_CK(cudaGetLastError());
            }
            PF_CK(launch_limbs<PF_IN_ATTN>(pf, st, nullptr, nullptr, pf->parts, nsplit, dim, dim, nv));
            {
                const int w[1] = {PF_WO}, col0[1] = {0};
                PF_CK(launch_gemm(pf, st, l, w, 1, dim, pf->parts, dim, col0, pf->ksplit_o, nv, false));
            }
            PF_CK(launch_limbs<PF_IN_NORM>(pf, st, pf->x, L.rms_ffn, pf->parts, pf->ksplit_o, dim, dim, nv));
            {
                const int w[2] = {PF_W1, PF_W3}, col0[2] = {0, hidden};
                PF_CK(launch_gemm(pf, st, l, w, 2, dim, pf->h13, 2 * hidden, col0, pf->ksplit_13, nv, true));
            }
            PF_CK(launch_limbs<PF_IN_SWIGLU>(pf, st, pf->h13, pf->h13 + hidden, nullptr, pf->ksplit_13, 2 * hidden, hidden, nv));
            {
                const int w[1] = {PF_W2}, col0[1] = {0};
                PF_CK(launch_gemm(pf, st, l, w, 1, hidden, pf->parts, dim, col0, pf->ksplit_2, nv, false));
            }
            pending = pf->ksplit_2;
        }
    }
    return cudaSuccess;
}

// Caches for n_seq sequences of seq_len positions each (replaces an earlier set).
cudaError_t prefill_batch_create(Prefill *pf, int n_seq, int seq_len)
{
    const PrefillModel &m = pf->m;
    if (n_seq < 1 || seq_len < 1 || seq_len > m.seq_len)
        return cudaErrorInvalidValue;
    const size_t per_seq = (size_t)m.n_layers * m.n_kv_heads * seq_len * m.head;
    auto drop = [&](void *ptr) {
        for (size_t i = 0; i < pf->owned.size(); ++i)
            if (pf->owned[i] == ptr) {
                cudaFree(ptr);
                pf->owned.erase(pf->owned.begin() + (long)i);
                return;
            }
    };
    for (auto &g : pf->step_graphs)
        cudaGraphExecDestroy(g.second);
    pf->step_graphs.clear();
    if (pf->bkc) {
        drop(pf->bkc);
        drop(pf->bvc);
        pf->bkc = pf->bvc = nullptr;
        pf->n_seq = 0;
    }
    PF_CK(pf_alloc(pf, &pf->bkc, per_seq * n_seq));
    PF_CK(pf_alloc(pf, &pf->bvc, per_seq * n_seq));
    if (!pf->meta) {
        PF_CK(pf_alloc(pf, &pf->meta, (size_t)4 * kT));
        PF_CK(pf_alloc(pf, &pf->xn, (size_t)kT * m.dim));
        PF_CK(pf_alloc(pf, &pf->logits, (size_t)kT * m.vocab));
        PF_CK(cudaHostAlloc(reinterpret_cast<void **>(&pf->meta_host), sizeof(int) * 4 * kT, cudaHostAllocDefault));
        PF_CK(cudaHostAlloc(reinterpret_cast<void **>(&pf->logits_host), sizeof(float) * (size_t)kT * m.vocab, cudaHostAllocDefault));
        PF_CK(cudaFuncSetAttribute(bd_classifier_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(2 * kClsStage * sizeof(float))));
    }
    pf->n_seq = n_seq;
    pf->seq_len_b = seq_len;
    return cudaSuccess;
}

// One decode step of n <= 64 (sequence, position, token) triples on one sweep over the weights; a sequence
// may appear several times with different positions (their K/V rows are all written before the attention).
// logits_out [n][vocab] and argmax_out [n] are host pointers (either may be null); blocks until done.
// Everything one step of n entries puts on the stream: tokens / positions / sequences in, all layers, classifier,
// arg-max ids out (pinned buffers on both ends, so the whole step can be captured into a graph).
static cudaError_t batch_enqueue(Prefill *pf, cudaStream_t st, int nv)
{
    const PrefillModel &m = pf->m;
    const int dim = m.dim, hidden = m.hidden, kvd = pf->kv_dim;
    PF_CK(cudaMemcpyAsync(pf->meta, pf->meta_host, sizeof(int) * 3 * kT, cudaMemcpyHostToDevice, st));
    const int *d_tok = pf->meta, *d_pos = pf->meta + kT, *d_seq = pf->meta + 2 * kT;
    int *d_arg = pf->meta + 3 * kT;
    const long long layer_stride = (long long)m.n_kv_heads * pf->seq_len_b * m.head;
    const long long seq_stride = layer_stride * m.n_layers;
    pf_embed_kernel<<<kT, 256, 0, st>>>(d_tok, nv, m.emb, dim, m.vocab, pf->x);
    ++pf->launches;
    PF_CK(cudaGetLastError());
    int pending = 0;
    for (int l = 0; l < m.n_layers; ++l) {
        const PrefillLayerDesc &L = m.layers[(size_t)l];
        PF_CK(launch_limbs<PF_IN_NORM>(pf, st, pf->x, L.rms_att, pf->parts, pending, dim, dim, nv));
        {
            const int w[3] = {PF_WQ, PF_WK, PF_WV}, col0[3] = {0, dim, dim + kvd};
            PF_CK(launch_gemm(pf, st, l, w, 3, dim, pf->qkv, pf->qkv_ld, col0, pf->ksplit_qkv, nv, true));
        }
        {
            PfRopeParams r{};
            r.qkv = pf->qkv; r.q = pf->q; r.k_cache = pf->bkc + l * layer_stride; r.v_cache = pf->bvc + l * layer_stride;
            r.rope_cos = m.rope_cos; r.rope_sin = m.rope_sin;
            r.dim = dim; r.kv_dim = kvd; r.head = m.head; r.seq_len = pf->seq_len_b; r.pos0 = 0; r.nvalid = nv;
            r.nparts = pf->ksplit_qkv;
            r.pos_of = d_pos; r.seq_of = d_seq; r.seq_stride = seq_stride;
            const dim3 grid((unsigned)kT, (unsigned)((pf->qkv_ld / 2 + 255) / 256));
            pf_rope_kv_kernel<<<grid, 256, 0, st>>>(r);
            ++pf->launches;
            PF_CK(cudaGetLastError());
        }
        {
            BdAttnParams a{};
            a.q = pf->q; a.k_cache = pf->bkc + l * layer_stride; a.v_cache = pf->bvc + l * layer_stride; a.seq_stride = seq_stride;
            a.pos_of = d_pos; a.seq_of = d_seq; a.parts = pf->parts;
            a.dim = dim; a.kv_mul = m.n_heads / m.n_kv_heads; a.seq_len = pf->seq_len_b; a.nvalid = nv;
            const dim3 grid((unsigned)m.n_heads, (unsigned)nv);
            if (m.head == 128)
                bd_attention_kernel<128><<<grid, 128, 0, st>>>(a);
            else
                bd_attention_kernel<64><<<grid, 128, 0, st>>>(a);
            ++pf->launches;
            PF_CK(cudaGetLastError());
        }
        PF_CK(launch_limbs<PF_IN_ATTN>(pf, st, nullptr, nullptr, pf->parts, 1, dim, dim, nv));
        {
            const int w[1] = {PF_WO}, col0[1] = {0};
            PF_CK(launch_gemm(pf, st, l, w, 1, dim, pf->parts, dim, col0, pf->ksplit_o, nv, false));
        }
        PF_CK(launch_limbs<PF_IN_NORM>(pf, st, pf->x, L.rms_ffn, pf->parts, pf->ksplit_o, dim, dim, nv));
        {
            const int w[2] = {PF_W1, PF_W3}, col0[2] = {0, hidden};
            PF_CK(launch_gemm(pf, st, l, w, 2, dim, pf->h13, 2 * hidden, col0, pf->ksplit_13, nv, true));
        }
        PF_CK(launch_limbs<PF_IN_SWIGLU>(pf, st, pf->h13, pf->h13 + hidden, nullptr, pf->ksplit_13, 2 * hidden, hidden, nv));
        {
            const int w[1] = {PF_W2}, col0[1] = {0};
            PF_CK(launch_gemm(pf, st, l, w, 1, hidden, pf->parts, dim, col0, pf->ksplit_2, nv, false));
        }
        pending = pf->ksplit_2;
    }
    bd_final_norm_kernel<<<kT, 256, 0, st>>>(pf->x, pf->parts, pending, m.rms_final, dim, nv, pf->xn);
    PF_CK(cudaGetLastError());
    bd_classifier_kernel<<<(m.vocab + kClsRows - 1) / kClsRows, kClsThreads, 2 * kClsStage * sizeof(float), st>>>(m.wcls, pf->xn, m.vocab, dim,
                                                                                                                 pf->logits);
    PF_CK(cudaGetLastError());
    bd_argmax_kernel<<<nv, 256, 0, st>>>(pf->logits, m.vocab, nv, d_arg);
    PF_CK(cudaGetLastError());
    pf->launches += 3;
    PF_CK(cudaMemcpyAsync(pf->meta_host + 3 * kT, d_arg, sizeof(int) * kT, cudaMemcpyDeviceToHost, st));
    return cudaSuccess;
}

cudaError_t prefill_batch_forward(Prefill *pf, cudaStream_t st, const int *tokens, const int *pos, const int *seq, int n, float *logits_out,
                                  int *argmax_out)
{
    const PrefillModel &m = pf->m;
    const int nv = n;
    for (int i = 0; i < kT; ++i) {
        pf->meta_host[i] = i < n ? tokens[i] : 0;
        pf->meta_host[kT + i] = i < n ? pos[i] : 0;
        pf->meta_host[2 * kT + i] = i < n ? seq[i] : 0;
    }
    // The step is about 330 launches of kernels that mostly run for a few microseconds: replayed as one graph per
    // entry count (grids and parameters depend on it; the caches and buffers stay where they are until
    // prefill_batch_create runs again).
    cudaGraphExec_t exec = nullptr;
    auto it = pf->step_graphs.find(nv);
    if (it != pf->step_graphs.end()) {
        exec = it->second;
    } else if (!pf->no_graph) {
        cudaGraph_t graph = nullptr;
        const unsigned long long before = pf->launches;
        if (cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) == cudaSuccess) {
            const cudaError_t ce = batch_enqueue(pf, st, nv);
            const cudaError_t ee = cudaStreamEndCapture(st, &graph);
            if (ce == cudaSuccess && ee == cudaSuccess && graph && cudaGraphInstantiate(&exec, graph, 0) == cudaSuccess) {
                pf->step_graphs[nv] = exec;
                pf->step_launches = pf->launches - before;
            } else {
                exec = nullptr;
                pf->no_graph = true;      // direct launches from now on
                cudaGetLastError();
            }
            if (graph)
                cudaGraphDestroy(graph);
        } else {
            pf->no_graph = true;
            cudaGetLastError();
        }
        pf->launches = before;
    }
    if (exec) {
        PF_CK(cudaGraphLaunch(exec, st));
        pf->launches += pf->step_launches;
    } else {
        PF_CK(batch_enqueue(pf, st, nv));
    }
    if (logits_out)
        PF_CK(cudaMemcpyAsync(pf->logits_host, pf->logits, sizeof(float) * (size_t)nv * m.vocab, cudaMemcpyDeviceToHost, st));
    PF_CK(cudaStreamSynchronize(st));
    if (logits_out)
        memcpy(logits_out, pf->logits_host, sizeof(float) * (size_t)nv * m.vocab);
    if (argmax_out)
        for (int i = 0; i < n; ++i)
            argmax_out[i] = pf->meta_host[3 * kT + i];
    return cudaSuccess;
}

int prefill_batch_sequences(const Prefill *pf)
{
    return pf ? pf->n_seq : 0;
}

int prefill_batch_seq_len(const Prefill *pf)
{
    return pf ? pf->seq_len_b : 0;
}

unsigned long long prefill_launches(const Prefill *pf)
{
    return pf ? pf->launches : 0;
}

}  // namespace l2j
