// Device-side building blocks for sm_100a: mbarrier + bulk-copy (TMA engine) wrappers with bounded
// waits, programmatic-dependent-launch controls, and the u8 -> f32 dot product used by the
// group-quantised matrix-vector kernels.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace l2j {

// ---------------------------------------------------------------------------------------------
// shared-memory barriers and bulk copies
// ---------------------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(bar), "r"(bytes)
                 : "memory");
}

// One poll of the barrier phase.  The hardware may suspend the thread for a bounded time inside
// the instruction; it always returns.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

__device__ __forceinline__ uint64_t global_timer_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Time base of the bounded waits: the SM's own cycle counter.  Reading %globaltimer costs on the order of a
// microsecond, which a wait loop that reads it pays on every poll that fails, i.e. on every hand-over inside a
// block; %clock64 is a register read.  A limit of t nanoseconds is taken as 2 t cycles (the SM clock is at
// most 2 GHz here, so the wait lasts at least t and at most about twice that at low clocks).
__device__ __forceinline__ long long sm_clock()
{
    long long c;
    asm volatile("mov.u64 %0, %%clock64;" : "=l"(c));
    return c;
}

// Bounded wait: gives up `timeout_ns` after the first failed poll and returns false; the caller
// records the fault in the device status word and carries on, so a lost copy can never hang the GPU.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, uint64_t timeout_ns)
{
    if (mbar_try_wait(bar, parity))
        return true;
    const long long c0 = sm_clock();
    const long long limit = (long long)(2 * timeout_ns);
    for (;;) {
        if (mbar_try_wait(bar, parity))
            return true;
        if (sm_clock() - c0 > limit)
            return false;
    }
}

// L2 eviction policy for data that is read exactly once per token (the weights).
__device__ __forceinline__ uint64_t policy_evict_first()
{
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

// Untiled bulk copy global -> shared; completion is signalled on `bar` as transferred bytes.
// dst, src and bytes must be multiples of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar, uint64_t policy)
{
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(dst),
        "l"(src), "r"(bytes), "r"(bar), "l"(policy)
        : "memory");
}

// 16-byte load through L2 that is only *issued* here: the asm is volatile, so later volatile asm
// (a barrier arrive, say) stays behind it in program order, and the data is waited for at first use.
__device__ __forceinline__ float4 ld_cg_f4_issue(const float *p)
{
    float4 v;
    asm volatile("ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}

// Asks the memory system to bring [src, src + bytes) into L2 (no destination, no completion signal).
// src and bytes must be multiples of 16.
__device__ __forceinline__ void bulk_prefetch_l2(const void *src, uint32_t bytes)
{
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}

// ---------------------------------------------------------------------------------------------
// programmatic dependent launch
// ---------------------------------------------------------------------------------------------

// Lets the next kernel in the stream start its prologue (weight prefetch) while this one runs.
__device__ __forceinline__ void pdl_launch_dependents()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Blocks until the previous kernel in the stream has finished and its writes are visible.
__device__ __forceinline__ void pdl_wait()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// hand-over counters between consecutive kernels
// ---------------------------------------------------------------------------------------------

__device__ __forceinline__ unsigned int ld_acquire_u32(const unsigned int *p)
{
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Publishes everything this thread (and, after a barrier, its block) wrote before: release + add.
__device__ __forceinline__ void red_release_add_u32(unsigned int *p, unsigned int v)
{
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// (value, sequence number) pairs of the tensor-parallel hand-over: one 8-byte store carries both, so the
// reader needs no fence; loads go to L2, where the peers' stores arrive.
__device__ __forceinline__ void st_pair(float2 *p, float v, int seq)
{
    asm volatile("st.volatile.global.v2.f32 [%0], {%1, %2};" ::"l"(p), "f"(v), "f"(__int_as_float(seq)) : "memory");
}

__device__ __forceinline__ float4 ld_pairs2(const float2 *p)
{
    float4 v;
    asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}

// Polls until the counter has reached `target` (wrap-around safe); gives up after timeout_ns and
// returns false, so a lost predecessor can never hang the GPU.
__device__ __forceinline__ bool counter_wait_bounded(const unsigned int *ctr, unsigned int target, uint64_t timeout_ns)
{
    if ((int)(ld_acquire_u32(ctr) - target) >= 0)
        return true;
    const long long c0 = sm_clock();
    const long long limit = (long long)(2 * timeout_ns);
    for (;;) {
        if ((int)(ld_acquire_u32(ctr) - target) >= 0)
            return true;
        if (sm_clock() - c0 > limit)
            return false;
    }
}

__device__ __forceinline__ void named_barrier_sync(int id, int nthreads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ---------------------------------------------------------------------------------------------
// arithmetic
// ---------------------------------------------------------------------------------------------

// Byte k of `w` as an exact float: place it in the low mantissa bits of 2^23, subtract 2^23.
// One permute on the integer pipe plus one add, instead of an int->float conversion.
template <int K>
__device__ __forceinline__ float u8_to_f32(uint32_t w)
{
#ifdef L2J_CVT_PLAIN
    return (float)((w >> (8 * K)) & 0xffu);
#else
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7440u | K)) - 8388608.0f;
#endif
}

// sum_j byte_j * x_j over the 16 bytes of `w`; two independent chains for ILP.
__device__ __forceinline__ float dot16_u8(const uint4 &w, const float (&x)[16])
{
    float a = 0.f, b = 0.f;
    a = fmaf(u8_to_f32<0>(w.x), x[0], a);
    b = fmaf(u8_to_f32<1>(w.x), x[1], b);
    a = fmaf(u8_to_f32<2>(w.x), x[2], a);
    b = fmaf(u8_to_f32<3>(w.x), x[3], b);
    a = fmaf(u8_to_f32<0>(w.y), x[4], a);
    b = fmaf(u8_to_f32<1>(w.y), x[5], b);
    a = fmaf(u8_to_f32<2>(w.y), x[6], a);
    b = fmaf(u8_to_f32<3>(w.y), x[7], b);
    a = fmaf(u8_to_f32<0>(w.z), x[8], a);
    b = fmaf(u8_to_f32<1>(w.z), x[9], b);
    a = fmaf(u8_to_f32<2>(w.z), x[10], a);
    b = fmaf(u8_to_f32<3>(w.z), x[11], b);
    a = fmaf(u8_to_f32<0>(w.w), x[12], a);
    b = fmaf(u8_to_f32<1>(w.w), x[13], b);
    a = fmaf(u8_to_f32<2>(w.w), x[14], a);
    b = fmaf(u8_to_f32<3>(w.w), x[15], b);
    return a + b;
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Reduces two values across the warp with five shuffles: afterwards lane 0 holds the sum of `a`
// over all lanes and lane 16 the sum of `b`.
__device__ __forceinline__ float warp_sum2(float a, float b, int lane)
{
    const bool hi = (lane & 16) != 0;
    float keep = hi ? b : a;
    float send = hi ? a : b;
    keep += __shfl_xor_sync(0xffffffffu, send, 16);
#pragma unroll
    for (int o = 8; o > 0; o >>= 1)
        keep += __shfl_xor_sync(0xffffffffu, keep, o);
    return keep;
}

// 1 / (1 + exp(-v)) with IEEE division and the accurate expf.
__device__ __forceinline__ float sigmoid_accurate(float v)
{
    return __fdiv_rn(1.0f, 1.0f + expf(-v));
}

}  // namespace l2j
