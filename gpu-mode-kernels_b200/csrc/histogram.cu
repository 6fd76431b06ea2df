// 256-bin histogram of bytes for sm_100a: the second task of the reference repository
// (pmpp_v2/histogram_py: `output = bincount(data, minlength=256)` on uint8 input, int64 output,
// reference.py:6-19).  HBM-bound byte work: 16-byte loads, two in flight per thread; private
// 256-bin tables per warp in shared memory (two replicas, chosen by lane parity, to halve bank and
// address conflicts); and, because the task's inputs make ONE value arbitrarily frequent
// (reference.py:36-39), every warp picks the value most common among its first 32 bytes as its
// candidate and counts that value with warp ballots into a register -- no atomic at all for it --
// while all other bytes go through shared-memory atomics.  One 64-bit global atomic per bin and block.
#include <cuda_runtime.h>
#include <stdint.h>

#include "a2a.h"

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kReplicas = 2;
constexpr int kBins = 256;

// One byte per lane: ballot-count the warp's candidate value, atomics for everything else.
__device__ __forceinline__ void count_byte(unsigned* table, unsigned v, bool valid, unsigned cand, unsigned& cand_count) {
    const bool is_cand = valid && v == cand;
    cand_count += __popc(__ballot_sync(0xffffffffu, is_cand));  // every lane keeps the same running count
    if (valid && !is_cand) atomicAdd(table + v, 1u);
}

__device__ __forceinline__ void count_vector(unsigned* table, const uint4& q, bool valid, unsigned cand, unsigned& cand_count) {
    const unsigned w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) count_byte(table, (w[a] >> (8 * b)) & 0xffu, valid, cand, cand_count);
}

__global__ void __launch_bounds__(kThreads) histogram256_kernel(const uint8_t* __restrict__ data, size_t n,
                                                                unsigned long long* __restrict__ out) {
    __shared__ unsigned tables[kWarps][kReplicas][kBins];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int i = tid; i < kWarps * kReplicas * kBins; i += kThreads) (&tables[0][0][0])[i] = 0u;
    __syncthreads();
    unsigned* table = tables[warp][lane & (kReplicas - 1)];
    // head: bytes before the first 16-byte boundary; body: 16-byte vectors; tail: the rest
    const uintptr_t addr = reinterpret_cast<uintptr_t>(data);
    size_t head = (16 - (addr & 15)) & 15;
    if (head > n) head = n;
    const size_t nvec = (n - head) / 16;
    const size_t tail0 = head + nvec * 16;
    const size_t gthreads = (size_t)gridDim.x * kThreads;
    const size_t gtid = (size_t)blockIdx.x * kThreads + tid;
    const uint4* vec = reinterpret_cast<const uint4*>(data + head);
    // every lane of a warp runs the same number of iterations (the ballots are warp-wide)
    const size_t rounds = (nvec + 2 * gthreads - 1) / (2 * gthreads);
    unsigned cand = 256u, cand_count = 0u;  // 256 = no candidate: every byte takes the atomic path
    for (size_t r = 0; r < rounds; ++r) {
        const size_t i0 = (2 * r) * gthreads + gtid, i1 = i0 + gthreads;
        const bool ok0 = i0 < nvec, ok1 = i1 < nvec;
        uint4 q0 = make_uint4(0u, 0u, 0u, 0u), q1 = q0;
        if (ok0) q0 = __ldg(vec + i0);
        if (ok1) q1 = __ldg(vec + i1);
        if (r == 0) {
            // the value most lanes hold in their first byte; worth a register only if it repeats
            const unsigned b0 = ok0 ? (q0.x & 0xffu) : 256u + lane;
            const unsigned peers = __match_any_sync(0xffffffffu, b0);
            const unsigned best = __reduce_max_sync(0xffffffffu, ((unsigned)__popc(peers) << 16) | b0);
            if ((best >> 16) >= 3u && (best & 0xffffu) < 256u) cand = best & 0xffu;
        }
        count_vector(table, q0, ok0, cand, cand_count);
        count_vector(table, q1, ok1, cand, cand_count);
    }
    if (blockIdx.x == 0) {  // the ragged ends: at most 15 + 15 bytes, one warp-wide pass each
        if (warp == 0) {
            const bool valid = (size_t)tid < head;
            count_byte(table, valid ? data[tid] : 0u, valid, cand, cand_count);
        } else if (warp == 1) {
            const size_t i = tail0 + (tid - 32);
            const bool valid = i < n;
            count_byte(table, valid ? data[i] : 0u, valid, cand, cand_count);
        }
    }
    if (lane == 0 && cand < 256u && cand_count) atomicAdd(tables[warp][0] + cand, cand_count);
    __syncthreads();
    unsigned long long sum = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w)
#pragma unroll
        for (int r = 0; r < kReplicas; ++r) sum += tables[w][r][tid];
    if (sum) atomicAdd(out + tid, sum);
}

}  // namespace

extern "C" int a2a_histogram256(const uint8_t* data, size_t n, int64_t* out, void* stream) {
    if (out == nullptr || (n > 0 && data == nullptr)) return A2A_ERR_CONFIG;
    if (reinterpret_cast<uintptr_t>(out) % 8 != 0) return A2A_ERR_CONFIG;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemsetAsync(out, 0, kBins * sizeof(int64_t), st);
    if (e != cudaSuccess) return -(int)e;
    if (n == 0) return A2A_OK;
    int dev = 0, sms = 0;
    if ((e = cudaGetDevice(&dev)) != cudaSuccess) return -(int)e;
    if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return -(int)e;
    // a multiple of the SM count; small inputs get fewer blocks (one vector per thread and round)
    const size_t want = (n / 32 + kThreads - 1) / kThreads;  // two vectors per thread and round
    size_t grid = (size_t)sms * 4;
    if (want < grid) grid = want < 1 ? 1 : want;
    histogram256_kernel<<<(unsigned)grid, kThreads, 0, st>>>(data, n, reinterpret_cast<unsigned long long*>(out));
    e = cudaGetLastError();
    return e == cudaSuccess ? A2A_OK : -(int)e;
}
