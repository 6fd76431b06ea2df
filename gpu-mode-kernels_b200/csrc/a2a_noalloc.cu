// a2a_route_noalloc -- routing for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need the
// routing tables: code running under a framework whose memory pool owns the whole device,
// plugins that are forbidden to touch the allocator after initialisation, latency-critical
// loops in which an allocation (a device-wide synchronising call) is not acceptable.  This
// entry point needs no context and allocates nothing: its working tables live in a
// file-scope device array that every GPU loading the library holds from load to exit
// (1 MiB), and the caller passes the input and both outputs.
//
// It computes exactly what a2a_route computes (see a2a_kernels.cuh): for every (token, k)
// pair the slot of its row inside the (expert, this source) slab, -1 for a pair whose
// expert is out of range or repeats an earlier k of its token, and the per-expert row
// counts.  The expert-by-token bitmap and its word prefix sums are kept in the static
// array instead of shared memory, which is also why this variant accepts more tokens per
// call than a context does.
//
// Limits and rules:
//   * num_experts <= 1024, num_tokens <= 4096, experts_per_token <= 32; anything larger is
//     rejected with A2A_ERR_CONFIG before any work is enqueued.
//   * The first call on a device looks up the device address of the array
//     (cudaGetSymbolAddress); make that first call outside any stream capture.
//   * All calls on one device share the one array and it keeps the previous call's
//     contents; the kernel clears the part it uses before using it.  Two calls whose
//     kernels overlap on the GPU (different streams, no dependency) race on it: serialise
//     them on one stream or with events.
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "a2a.h"

namespace {

constexpr int kMaxExperts = 1024;
constexpr int kMaxTokens = 4096;
constexpr int kMaxTopK = 32;
constexpr int kMaxWords = kMaxTokens / 32;  // bitmap words per expert
constexpr int kThreads = 1024;
constexpr int kMaxDevices = 64;

// [0, W*E): bitmap, bit t%32 of word (t/32)*E + e set iff token t uses expert e
// [kMaxWords*kMaxExperts, +W*E): number of set bits in the words before w, per expert
static __device__ __align__(256) unsigned g_route_scratch[2 * kMaxWords * kMaxExperts];

__global__ void __launch_bounds__(kThreads) route_noalloc_kernel(unsigned* scratch, const int* __restrict__ idx, int T,
                                                                int E, int K, int* __restrict__ slots,
                                                                int* __restrict__ counts) {
    unsigned* bits = scratch;
    int* wpre = reinterpret_cast<int*>(scratch + kMaxWords * kMaxExperts);
    const int tid = threadIdx.x;
    const int Wc = (T + 31) >> 5;
    // the array keeps the previous call's bits: clear what this call will read
    for (int i = tid; i < Wc * E; i += kThreads) bits[i] = 0u;
    __syncthreads();
    for (int t = tid; t < T; t += kThreads) {
        const int* row = idx + (size_t)t * K;
        for (int k = 0; k < K; ++k) {
            const int e = row[k];
            if (e >= 0 && e < E) atomicOr(bits + (t >> 5) * E + e, 1u << (t & 31));
        }
    }
    __syncthreads();
    for (int e = tid; e < E; e += kThreads) {
        int run = 0;
        for (int w = 0; w < Wc; ++w) {
            wpre[w * E + e] = run;
            run += __popc(bits[w * E + e]);
        }
        counts[e] = run;
    }
    __syncthreads();
    for (int t = tid; t < T; t += kThreads) {
        const int* row = idx + (size_t)t * K;
        for (int k = 0; k < K; ++k) {
            const int e = row[k];
            bool valid = (e >= 0 && e < E);
            for (int kk = 0; kk < k && valid; ++kk) valid = (row[kk] != e);
            int s = -1;
            if (valid) {
                const int w = t >> 5;
                s = wpre[w * E + e] + __popc(bits[w * E + e] & ((1u << (t & 31)) - 1u));
            }
            slots[(size_t)t * K + k] = s;
        }
    }
}

// Device address of the static array, looked up once per device with that device current.
// In host code the array's name is only a handle for the runtime, never a pointer a kernel
// may be given.
unsigned* g_scratch_addr[kMaxDevices];
std::mutex g_setup_mutex;

int scratch_for_current_device(unsigned** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return -(int)e;
    if (dev < 0 || dev >= kMaxDevices) return A2A_ERR_CONFIG;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_addr[dev] == nullptr) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_route_scratch);
        if (e != cudaSuccess) return -(int)e;
        g_scratch_addr[dev] = static_cast<unsigned*>(ptr);
    }
    *out = g_scratch_addr[dev];
    return A2A_OK;
}

}  // namespace

extern "C" int a2a_route_noalloc(const int32_t* topk_idx, int num_tokens, int num_experts, int experts_per_token,
                                 int32_t* slots_out, int32_t* send_counts_out, void* stream) {
    if (num_experts < 1 || num_experts > kMaxExperts) return A2A_ERR_CONFIG;
    if (num_tokens < 0 || num_tokens > kMaxTokens) return A2A_ERR_CONFIG;
    if (experts_per_token < 1 || experts_per_token > kMaxTopK) return A2A_ERR_CONFIG;
    if (send_counts_out == nullptr || (num_tokens > 0 && (topk_idx == nullptr || slots_out == nullptr)))
        return A2A_ERR_CONFIG;
    unsigned* scratch = nullptr;
    const int r = scratch_for_current_device(&scratch);
    if (r != A2A_OK) return r;
    route_noalloc_kernel<<<1, kThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        scratch, topk_idx, num_tokens, num_experts, experts_per_token, slots_out, send_counts_out);
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? A2A_OK : -(int)e;
}
