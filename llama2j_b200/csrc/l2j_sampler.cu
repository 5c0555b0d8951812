// Temperature / top-p token selection on the device, reproducing the reference's host-side Sampler bit for
// bit, so that `--temp 0.9 --seed S` chooses the tokens the Java program would choose from the same logits
// and only the chosen id (4 bytes) crosses PCIe instead of the 128 KB of logits.
//
// Reference (paths relative to src/main/java/com/lastbot/llama2j/):
//   Run.java:643-665        logits /= temperature; FindMax.call; ExpSumNormalize.call (exp in double, the sum
//                           one sequential float accumulator); Sampler.sample or Sampler.sample_topp
//   Sampler.java:20-44      java.util.Random.nextFloat() (48-bit LCG), the cumulative walk
//   Sampler.java:76-120     top-p: candidates >= (1 - topp) / (n - 1) in index order into the FIRST n0 entries of
//                           a ProbIndex array that lives as long as the Sampler, a STABLE descending sort of the
//                           WHOLE array (so entries that earlier calls left beyond n0 take part), the
//                           cumulative cut, the draw
//
// One block.  Everything whose result depends on the order of float additions (the softmax sum, the two
// cumulative walks) is done by one thread in the reference's order, out of shared memory; the rest (division,
// exponentials, candidate compaction, the sort) is parallel and order-preserving.  The sort is a stable
// least-significant-digit radix sort on the bit pattern of the (non-negative) probabilities, which orders
// exactly as ProbIndex.compareTo does.

#include "l2j_device.cuh"
#include "l2j_internal.h"

#include <cfloat>
#include <cmath>

namespace l2j {

namespace {

constexpr int kSampThreads = 1024;
constexpr int kRadixBits = 4, kRadix = 1 << kRadixBits, kRadixPasses = 32 / kRadixBits;   // 8 passes: the data ends where it began

__device__ __forceinline__ int rng_next(unsigned long long &rng, int bits)
{
    rng = (rng * 0x5DEECE66DULL + 0xBULL) & ((1ULL << 48) - 1ULL);
    return (int)((long long)rng >> (48 - bits));
}

__device__ __forceinline__ float rng_next_float(unsigned long long &rng)
{
    return __fdiv_rn((float)rng_next(rng, 24), 16777216.0f);
}

// Exclusive prefix sum of one value per thread over the block; returns the thread's offset, `total` the sum.
__device__ __forceinline__ int block_exclusive_scan(int v, int *warp_sums, int &total)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o)
            inc += t;
    }
    if (lane == 31)
        warp_sums[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        int w = warp_sums[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o)
                w += t;
        }
        warp_sums[lane] = w;   // inclusive sums of the warps
    }
    __syncthreads();
    total = warp_sums[31];
    const int base = warp > 0 ? warp_sums[warp - 1] : 0;
    __syncthreads();
    return base + inc - v;
}

}  // namespace

__global__ void __launch_bounds__(kSampThreads, 1) sample_kernel(const __grid_constant__ SampleParams sp)
{
    extern __shared__ __align__(16) unsigned char ssm[];
    float *p = reinterpret_cast<float *>(ssm);                                    // n floats
    unsigned int *offs = reinterpret_cast<unsigned int *>(ssm + (size_t)((sp.n + 3) & ~3) * 4);   // kRadix * 1024
    __shared__ int warp_sums[32];
    __shared__ float s_red[32];
    __shared__ float s_bcast;
    __shared__ int s_n0;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n = sp.n;
    const int per = (n + kSampThreads - 1) / kSampThreads;       // elements per thread of the order-preserving steps
    const int lo = min(n, tid * per), hi = min(n, lo + per);

    // ---- logits / temperature, their maximum (Run.java:645-652, FindMax.call)
    float mx = -FLT_MAX;
    for (int i = tid; i < n; i += kSampThreads) {
        const float v = __fdiv_rn(sp.logits[i], sp.temperature);
        p[i] = v;
        mx = fmaxf(mx, v);
    }
    mx = warp_max(mx);
    if (lane == 0)
        s_red[warp] = mx;
    __syncthreads();
    mx = warp_max(s_red[lane]);
    // ---- exp in double, one sequential float sum, division (ExpSumNormalize.call, ExpSumNormalize.java:25-38)
    for (int i = tid; i < n; i += kSampThreads)
        p[i] = (float)exp((double)__fsub_rn(p[i], mx));
    __syncthreads();
    if (tid == 0) {
        float sum = 0.0f;
        int i = 0;
        for (; i + 8 <= n; i += 8) {
            const float4 a = *reinterpret_cast<const float4 *>(p + i), b = *reinterpret_cast<const float4 *>(p + i + 4);
            sum = __fadd_rn(sum, a.x); sum = __fadd_rn(sum, a.y); sum = __fadd_rn(sum, a.z); sum = __fadd_rn(sum, a.w);
            sum = __fadd_rn(sum, b.x); sum = __fadd_rn(sum, b.y); sum = __fadd_rn(sum, b.z); sum = __fadd_rn(sum, b.w);
        }
        for (; i < n; ++i)
            sum = __fadd_rn(sum, p[i]);
        s_bcast = sum;
    }
    __syncthreads();
    const float sum = s_bcast;
    if (sum != 0.0f)
        for (int i = tid; i < n; i += kSampThreads)
            p[i] = __fdiv_rn(p[i], sum);
    __syncthreads();
    for (int i = tid; i < n; i += kSampThreads)
        sp.logits[i] = p[i];   // the reference turns the logits into probabilities in place

    unsigned long long rng = sp.st->rng;
    int token = n - 1;
    if ((double)sp.topp > 0.999) {   // Run.java:658 compares the float with the double literal
        // ---- Sampler.sample (Sampler.java:33-44)
        if (tid == 0) {
            const float r = rng_next_float(rng);
            float cdf = 0.0f;
            for (int i = 0; i < n; ++i) {
                cdf = __fadd_rn(cdf, p[i]);
                if (r < cdf) {
                    token = i;
                    break;
                }
            }
        }
    } else {
        // ---- Sampler.sample_topp (Sampler.java:76-120)
        const float cutoff = __fdiv_rn(__fsub_rn(1.0f, sp.topp), (float)(n - 1));
        int cnt = 0;
        for (int i = lo; i < hi; ++i)
            cnt += p[i] >= cutoff ? 1 : 0;
        int total = 0;
        int at = block_exclusive_scan(cnt, warp_sums, total);
        for (int i = lo; i < hi; ++i) {
            if (p[i] >= cutoff) {           // candidates in index order into the first n0 entries
                sp.prob[0][at] = p[i];
                sp.index[0][at] = i;
                ++at;
            }
        }
        if (tid == 0)
            s_n0 = total;
        __syncthreads();
        // stable descending sort of the whole array: least-significant-digit radix sort on ~bits(prob)
        for (int pass = 0; pass < kRadixPasses; ++pass) {
            const float *src_p = sp.prob[pass & 1];
            const int *src_i = sp.index[pass & 1];
            float *dst_p = sp.prob[(pass + 1) & 1];
            int *dst_i = sp.index[(pass + 1) & 1];
            const int shift = pass * kRadixBits;
            unsigned int cntd[kRadix];
#pragma unroll
            for (int d = 0; d < kRadix; ++d)
                cntd[d] = 0;
            for (int i = lo; i < hi; ++i) {
                const unsigned int d = ((~__float_as_uint(src_p[i])) >> shift) & (kRadix - 1);
#pragma unroll
                for (int q = 0; q < kRadix; ++q)
                    cntd[q] += (d == (unsigned)q) ? 1u : 0u;
            }
#pragma unroll
            for (int d = 0; d < kRadix; ++d)
                offs[d * kSampThreads + tid] = cntd[d];
            __syncthreads();
            // exclusive scan over the kRadix * 1024 counters in digit-major order: thread t owns entries 16 t .. 16 t + 15
            unsigned int local[kRadix];
            int run = 0;
#pragma unroll
            for (int q = 0; q < kRadix; ++q) {
                local[q] = offs[tid * kRadix + q];
                run += (int)local[q];
            }
            int tot2 = 0;
            int base = block_exclusive_scan(run, warp_sums, tot2);
#pragma unroll
            for (int q = 0; q < kRadix; ++q) {
                offs[tid * kRadix + q] = (unsigned)base;
                base += (int)local[q];
            }
            __syncthreads();
#pragma unroll
            for (int d = 0; d < kRadix; ++d)
                cntd[d] = offs[d * kSampThreads + tid];
            for (int i = lo; i < hi; ++i) {           // in order: equal keys keep their order
                const float pv = src_p[i];
                const unsigned int d = ((~__float_as_uint(pv)) >> shift) & (kRadix - 1);
                unsigned int pos = 0;
#pragma unroll
                for (int q = 0; q < kRadix; ++q) {
                    if (d == (unsigned)q) {
                        pos = cntd[q];
                        cntd[q] = pos + 1;
                    }
                }
                dst_p[pos] = pv;
                dst_i[pos] = src_i[i];
            }
            __syncthreads();
        }
        // ---- the cumulative cut and the draw, by one thread in the reference's order
        const int n0 = s_n0;
        for (int i = tid; i < n0; i += kSampThreads)
            p[i] = sp.prob[0][i];
        __syncthreads();
        if (tid == 0) {
            float cumulative = 0.0f;
            int last_idx = n0 - 1;
            for (int i = 0; i < n0; ++i) {
                cumulative = __fadd_rn(cumulative, p[i]);
                if (cumulative > sp.topp) {
                    last_idx = i;
                    break;
                }
            }
            const float r = __fmul_rn(rng_next_float(rng), cumulative);
            float cdf = 0.0f;
            token = last_idx >= 0 ? sp.index[0][last_idx] : 0;
            for (int i = 0; i <= last_idx; ++i) {
                cdf = __fadd_rn(cdf, p[i]);
                if (r < cdf) {
                    token = sp.index[0][i];
                    break;
                }
            }
        }
    }
    if (tid == 0) {
        sp.st->rng = rng;
        sp.st->token = token;
    }
}

size_t sample_smem_bytes(int n)
{
    return (size_t)((n + 3) & ~3) * 4 + (size_t)kRadix * kSampThreads * 4;
}

cudaError_t prepare_sampler(int n)
{
    return cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sample_smem_bytes(n));
}

cudaError_t launch_sample(cudaStream_t stream, const SampleParams &sp)
{
    sample_kernel<<<1, kSampThreads, sample_smem_bytes(sp.n), stream>>>(sp);
    return cudaGetLastError();
}

}  // namespace l2j
