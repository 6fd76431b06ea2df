// Device-side building blocks shared by the all-to-all kernels: parameter block,
// system-scope flag operations with bounded waits, 16-byte row access, block scan.
//
// Memory-ordering protocol used throughout (producer on GPU A, consumer on GPU B):
//   producer threads: plain stores to B's memory -> __threadfence_system() ->
//   block barrier -> one thread: atomic ticket on A; the block that draws the last
//   ticket fences again and writes the flag with st.release.sys into B's memory.
//   consumer: ld.acquire.sys on its own flag until it carries this call's epoch
//   (bounded by a wall-clock budget), block barrier, then plain loads.
// Flags carry a monotonically increasing call number ("epoch"), are never reset,
// and every (source, destination) pair has its own flag word on its own 128-byte line.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "a2a.h"

namespace a2a {

constexpr int kFlagStride = 32;  // uint32 words between two flags = 128 bytes
enum FlagKind : int { kFlagDispatch = 0, kFlagExpert = 1, kFlagBarrier = 2, kNumFlagKinds = 3 };
enum Phase : int { kPhaseRoute = 1, kPhaseSend = 2, kPhaseRecv = 3, kPhaseExpert = 4, kPhaseCombine = 5, kPhaseBarrier = 6 };

// Everything a kernel needs, passed by value (lives in the constant bank).
struct DevParams {
    uint8_t* peer[A2A_MAX_WORLD];  // base of every rank's symmetric region as mapped here; peer[rank] is our own
    // byte offsets inside a symmetric region (identical on every rank)
    size_t off_rows;        // [L][ws][T_max][H] elements: slab (l, src) holds the rows src sent to local expert l
    size_t off_meta;        // [L][ws][T_max] int32: (token << 8) | k of every row
    size_t off_counts;      // [ws][L] int32: rows source s sent to local expert l in the current call
    size_t off_flags;       // [kNumFlagKinds][ws][kFlagStride] uint32 epochs
    size_t off_stage;       // [ws][T_max][stage_row_bytes]: one wire row per (source, token)   (DEDUP / FP8)
    size_t off_stage_meta;  // [ws][T_max][K] int32: (local_expert << 16 | slot) or -1 per k   (DEDUP / FP8)
    int stage_row_bytes;
    int rank, ws, E, K, H, T_max, L;
    int T;                  // tokens of this rank in the current call
    uint32_t epoch;
    long long timeout_ns;
    // local scratch of this rank
    int* slot;              // [T_max*K] slot of pair (t,k) inside slab (expert, this rank), -1 = dropped
    int* send_counts;       // [E]
    int* expert_count;      // [L] rows per local expert summed over sources
    uint32_t* tickets;      // [8] block-arrival counters, one per kernel kind
    a2a_status_t* status;
    // caller tensors of the current call
    const int* idx;
    const void* x;
    const float* w;
    void* y;
};

__device__ __forceinline__ long long global_ns() {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ int ld_volatile_i32(const int* p) {
    int v;
    asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Read-only 16-byte load of caller input (never written while the kernel runs).
__device__ __forceinline__ uint4 ld_input(const uint4* p) { return __ldg(p); }

// 16-byte load of data another GPU (or an earlier phase) produced: skip L1, one use.
__device__ __forceinline__ uint4 ld_stream(const uint4* p) { return __ldcg(p); }

// 16-byte store that will not be re-read by this SM.
__device__ __forceinline__ void st_stream(uint4* p, uint4 v) { __stcg(p, v); }

__device__ __forceinline__ void record_error(a2a_status_t* st, int code, int rank, int peer, int phase,
                                             uint32_t epoch, int detail) {
    if (atomicCAS(&st->code, 0, code) == 0) {
        st->rank = rank;
        st->peer = peer;
        st->phase = phase;
        st->epoch = epoch;
        st->detail = detail;
        __threadfence();
    }
}

__device__ __forceinline__ uint32_t* flag_ptr(uint8_t* region_base, size_t off_flags, int kind, int index) {
    return reinterpret_cast<uint32_t*>(region_base + off_flags) + ((size_t)kind * A2A_MAX_WORLD + index) * kFlagStride;
}

// Spin until *flag has reached `epoch` (wrap-safe).  Gives up after timeout_ns, or as
// soon as any thread of this rank has recorded an error, and returns false.
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t epoch, const DevParams& p, int phase, int peer) {
    if ((int32_t)(ld_acquire_sys(flag) - epoch) >= 0) return true;
    const long long t0 = global_ns();
    unsigned backoff = 32;
    for (;;) {
        if ((int32_t)(ld_acquire_sys(flag) - epoch) >= 0) return true;
        if (ld_volatile_i32(&p.status->code) != 0) return false;
        if (global_ns() - t0 > p.timeout_ns) {
            record_error(p.status, A2A_ERR_TIMEOUT, p.rank, peer, phase, epoch, 0);
            return false;
        }
        __nanosleep(backoff);
        if (backoff < 256) backoff <<= 1;
    }
}

// All threads of the block call this after their last store of the kernel.  Returns
// true in exactly one block of the grid: the one that arrived last, after which every
// store of every block is ordered before whatever that block publishes next.
__device__ __forceinline__ bool grid_arrive_last(uint32_t* ticket) {
    __shared__ int s_last;
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t t = atomicAdd(ticket, 1u);
        const int last = (t == gridDim.x - 1);
        if (last) *ticket = 0;  // everyone has arrived: re-arm for the next launch
        __threadfence_system();
        s_last = last;
    }
    __syncthreads();
    return s_last != 0;
}

// Exclusive prefix sum over n <= 4*blockDim.x ints held in shared memory `a`
// (in place; a[n] receives the total).  blockDim.x must be 256.
__device__ __forceinline__ void block_exclusive_scan(int* a, int n) {
    __shared__ int s_warp[8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int per = (n + 255) / 256;
    const int lo = tid * per;
    int sum = 0;
    __syncthreads();  // a[] was filled by other threads
    for (int i = 0; i < per; ++i)
        if (lo + i < n) sum += a[lo + i];
    int inc = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int v = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += v;
    }
    if (lane == 31) s_warp[warp] = inc;
    __syncthreads();
    int base = 0;
    for (int w = 0; w < warp; ++w) base += s_warp[w];
    int run = base + inc - sum;
    for (int i = 0; i < per; ++i)
        if (lo + i < n) {
            int v = a[lo + i];
            a[lo + i] = run;
            run += v;
        }
    if (tid == 255) a[n] = base + inc;
    __syncthreads();
}

// Largest i in [0, n) with prefix[i] <= r, given prefix is non-decreasing and prefix[n] > r.
__device__ __forceinline__ int upper_slab(const int* prefix, int n, int r) {
    int lo = 0, hi = n;
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (prefix[mid] <= r) lo = mid; else hi = mid;
    }
    return lo;
}

// ---- element types ---------------------------------------------------------
template <typename T> struct Vec2;
template <> struct Vec2<__nv_bfloat16> {
    using type = __nv_bfloat162;
    static __device__ __forceinline__ float2 to_float2(type v) { return __bfloat1622float2(v); }
    static __device__ __forceinline__ type from_float2(float2 v) { return __float22bfloat162_rn(v); }
};
template <> struct Vec2<__half> {
    using type = __half2;
    static __device__ __forceinline__ float2 to_float2(type v) { return __half22float2(v); }
    static __device__ __forceinline__ type from_float2(float2 v) { return __float22half2_rn(v); }
};

// 8 elements (16 bytes) <-> 8 floats
template <typename T>
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    using V = typename Vec2<T>::type;
    const V* h = reinterpret_cast<const V*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 t = Vec2<T>::to_float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}

template <typename T>
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    using V = typename Vec2<T>::type;
    uint4 v;
    V* h = reinterpret_cast<V*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = Vec2<T>::from_float2(make_float2(f[2 * i], f[2 * i + 1]));
    return v;
}

}  // namespace a2a
