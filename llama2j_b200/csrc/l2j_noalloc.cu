// l2j_k_attention_noalloc: the attention kernel for callers that are not allowed to allocate.
//
// Some hosts of this library run inside a memory budget they must not exceed or even touch: a
// serving process that has handed its whole device-memory pool to another allocator, or a real-time
// loop where cudaMalloc's implicit device synchronisation and its unbounded latency are not
// acceptable once the stream is running.  The regular attention entry point allocates its split
// scratch (and staging buffers) on every call.  This one allocates nothing: its scratch is the
// fixed array below, which every GPU that loads the library holds from load to exit, and the
// caller brings inputs and outputs as device pointers.

#include "../../include/l2j_b200.h"
#include "l2j_internal.h"

#include <cstdio>
#include <mutex>

using namespace l2j;

namespace {

// Largest problem the fixed scratch can serve.
constexpr int kNaMaxHeads = 128;
constexpr int kNaMaxHead = 128;
constexpr int kNaMaxSplit = 32;
constexpr size_t kNaPartFloats = (size_t)kNaMaxHeads * kNaMaxSplit * (kNaMaxHead + 2);
constexpr size_t kNaScratchBytes = kNaPartFloats * sizeof(float) + kNaMaxHeads * sizeof(unsigned int);   // about 2.1 MB

// The scratch itself: split partials (m, l, o[head]) per (head, split), then one arrival counter
// per head.  In host code this name is only a stand-in for the symbol; the address a kernel can use
// comes from cudaGetSymbolAddress, once per device.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNaScratchBytes];

constexpr int kNaMaxDevices = 64;
std::mutex g_na_mu;
void *g_na_ptr[kNaMaxDevices] = {nullptr};
int g_na_sms[kNaMaxDevices] = {0};
thread_local char g_na_error[256] = "";

int na_fail(int code, const char *msg, cudaError_t e = cudaSuccess)
{
    if (e != cudaSuccess)
        snprintf(g_na_error, sizeof(g_na_error), "%s: %s", msg, cudaGetErrorString(e));
    else
        snprintf(g_na_error, sizeof(g_na_error), "%s", msg);
    return code;
}

}  // namespace

extern "C" const char *l2j_noalloc_last_error(void)
{
    return g_na_error;
}

extern "C" int l2j_k_attention_noalloc(int device, const float *q_dev, const float *k_cache_dev, const float *v_cache_dev,
                                       int pos, int n_heads, int n_kv_heads, int head_size, int seq_len, float *out_dev,
                                       void *stream)
{
    g_na_error[0] = 0;
    if (!q_dev || !k_cache_dev || !v_cache_dev || !out_dev)
        return na_fail(L2J_E_INVALID, "null device pointer");
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || head_size <= 0 || head_size % 4 != 0 || seq_len <= 0 ||
        pos < 0 || pos >= seq_len)
        return na_fail(L2J_E_INVALID, "bad shape or position");
    if (n_heads > kNaMaxHeads || head_size > kNaMaxHead)
        return na_fail(L2J_E_INVALID, "problem exceeds the fixed scratch: at most 128 heads of at most 128 floats");
    if (device < 0 || device >= kNaMaxDevices)
        return na_fail(L2J_E_INVALID, "device index out of range");
    // The launch needs `device` current; the caller's own current device is put back on every way out.
    struct DeviceGuard {
        int prev = -1;
        ~DeviceGuard()
        {
            if (prev >= 0)
                cudaSetDevice(prev);
        }
    } guard;
    int current = -1;
    cudaError_t e = cudaGetDevice(&current);
    if (e != cudaSuccess)
        return na_fail(L2J_E_CUDA, "cudaGetDevice failed", e);
    if (current != device) {
        e = cudaSetDevice(device);
        if (e != cudaSuccess)
            return na_fail(L2J_E_CUDA, "cudaSetDevice failed", e);
        guard.prev = current;
    }

    void *scratch = nullptr;
    int sms = 0;
    {
        // First call on this device: resolve the device address of the scratch symbol.  Do this
        // outside any stream capture (the query is not a stream operation).
        std::lock_guard<std::mutex> lock(g_na_mu);
        if (!g_na_ptr[device]) {
            void *ptr = nullptr;
            e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
            if (e != cudaSuccess || !ptr)
                return na_fail(L2J_E_CUDA, "cudaGetSymbolAddress failed", e);
            int n = 0;
            e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device);
            if (e != cudaSuccess || n <= 0)
                return na_fail(L2J_E_CUDA, "cudaDeviceGetAttribute failed", e);
            g_na_ptr[device] = ptr;
            g_na_sms[device] = n;
        }
        scratch = g_na_ptr[device];
        sms = g_na_sms[device];
    }

    AttnParams p{};
    p.nsplit = choose_nsplit(sms, n_heads, seq_len);   // the split of l2j_k_attention: same partial sums, same bits
    static_assert(kNaMaxSplit >= 32, "choose_nsplit returns at most 32 splits");
    p.q = q_dev;
    p.k_cache = k_cache_dev;
    p.v_cache = v_cache_dev;
    p.out = out_dev;
    p.out_reps = 1;
    p.out_stride = 0;
    p.part = static_cast<float *>(scratch);
    p.counters = reinterpret_cast<unsigned int *>(static_cast<unsigned char *>(scratch) + kNaPartFloats * sizeof(float));
    p.state = nullptr;              // never read: the position is passed explicitly
    p.n_heads = n_heads;
    p.kv_mul = n_heads / n_kv_heads;
    p.head = head_size;
    p.seq_len = seq_len;
    p.pos_override = pos;

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // The array keeps whatever the previous call left; the arrival counters must start at zero.
    e = cudaMemsetAsync(p.counters, 0, sizeof(unsigned int) * (size_t)n_heads, s);
    if (e != cudaSuccess)
        return na_fail(L2J_E_CUDA, "cudaMemsetAsync failed", e);
    LaunchCfg lc{s, false, sms};
    e = launch_attention(lc, p);
    if (e != cudaSuccess)
        return na_fail(L2J_E_CUDA, "kernel launch failed", e);
    return L2J_OK;
}
