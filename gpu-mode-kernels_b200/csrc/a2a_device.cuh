// Device-side building blocks shared by the all-to-all kernels: parameter block,
// system-scope flag operations with bounded waits, 16-byte row access, block scan,
// element conversions (bf16 / fp16 / fp8 e4m3).
//
// Synchronisation.  System-scope fences are the scarce resource on this machine: a
// B200 retires them at roughly 100-150 per microsecond for the whole chip (740 blocks
// executing one fence.sys each take ~6.5 us; four each take ~31 us), whereas gpu-scope
// fences are nearly free (a fence.gpu after every row costs ~1 us over 2048 rows).  So:
//   * blocks of one GPU synchronise among themselves at gpu scope only: after its last
//     store of a phase a block meets at a barrier, ONE thread fences at gpu scope and draws
//     an atomic ticket;
//   * the block that draws the last ticket is the phase's publisher: for the consumers on
//     its own GPU a gpu-scope release of a local word, for the peers one fence.sys and then
//     relaxed system-scope stores of this call's epoch into one flag word per peer;
//   * on the consumer GPU one "watcher" thread per flag polls it with relaxed system-scope
//     loads (strong, L1-bypassing; an acquire load per poll would run a fence per
//     iteration), takes ONE system-scope acquire fence once the flag has arrived (so the
//     producer's release and this acquire are a morally strong pair under the PTX model)
//     and re-publishes the flag in a local word with a gpu-scope release; everybody else
//     waits on the local word at gpu scope and reads the rows with L1-bypassing loads.
//     Only the watcher threads (at most one per peer and flag kind) ever execute a
//     system-scope fence on the consumer side: a fence.sys in every waiting block is a
//     flush round trip over NVLink that queues behind the row traffic.
// The PTX memory model makes causality order transitive across edges of different scope,
// so a row stored by any block of GPU A is visible to any block of GPU B that has seen
// B's local word, with a handful of system fences per GPU and call instead of thousands
// (none at all on a single GPU).
// Flags carry a monotonically increasing call number ("epoch"), are never reset, and
// every (source, destination) pair has its own flag word on its own 128-byte line.
// Every wait is bounded by a wall-clock budget; on expiry the kernel records
// A2A_ERR_TIMEOUT and returns normally.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "a2a.h"

namespace a2a {

constexpr int kThreads = 256;    // every kernel of the path runs 256-thread blocks
constexpr int kFlagStride = 32;  // uint32 words between two flags = 128 bytes
constexpr int kFp8Block = 128;   // elements sharing one fp32 scale
constexpr int kMaxChunks = 4;    // token chunks a call is pipelined in (whole 32-token bitmap words each)
constexpr int kStageBytes = 16384;  // one stage of a sender block's shared-memory ring (a row piece)
constexpr int kStages = 6;          // stages of that ring: four bulk loads and two bulk stores in flight
constexpr unsigned kNoEntry = 0xffffffffu;  // record entry of a (token, k) pair that has no row on the destination
enum FlagKind : int { kFlagDispatch = 0, kFlagExpert = 1, kFlagBarrier = 2, kNumFlagKinds = 3 };
enum Phase : int { kPhaseRoute = 1, kPhaseSend = 2, kPhaseRecv = 3, kPhaseExpert = 4, kPhaseCombine = 5, kPhaseBarrier = 6 };
// In-kernel trace: thread 0 of every block stamps these points with the SM cycle counter
// (slot 0 additionally holds the nanosecond global timer so blocks can be aligned).
enum Ticket : int { kTicketSend = 0, kTicketExpert = 1 };
// The phase-by-phase kernels stamp slots 1..7; the pipelined kernel additionally stamps, per
// position i of its source / destination order, when a sender block finished destination i
// (kStampDestDone + i), when an expert block saw source i's rows (kStampSourceSeen + i) and
// when it was through with them (kStampSourceDone + i).  kStampRole tells what the block was.
enum Stamp : int {
    kStampGlobalNs = 0, kStampStart, kStampRouted, kStampSent, kStampDispatchSeen, kStampExpertDone,
    kStampExpertSeen, kStampCombineDone, kStampRole = kStampRouted /* pipelined: what the block was */,
    kStampSourceSeen = 8, kStampSourceDone = 16, kStampDestDone = 24,
    // finer steps inside a role, in slots that role does not use otherwise: a router block stamps
    // kStampStep + {0 bitmap cleared, 1 bitmap built, 2 scanned, 3 records written}; a sender block
    // kStampSetup + {0 token lists built, 1 first load issued, 2 first store issued}
    kStampStep = 24, kStampSetup = 8,
    kNumStamps = 32
};
enum Role : int { kRoleSender = 1, kRoleExpert = 2, kRoleRouter = 4, kRoleWatcher = 8 };

// Everything a kernel needs, passed by value (lives in the constant bank).
struct DevParams {
    uint8_t* peer[A2A_MAX_WORLD];  // base of every rank's symmetric region as mapped here; peer[rank] is our own
    // byte offsets inside a symmetric region (identical on every rank)
    size_t off_rows;        // [L][ws][T_max][H] elements: slab (l, src) holds the rows src sent to local expert l
    size_t off_meta;        // [L][ws][T_max] int32: (token << 8) | k of every row
    size_t off_counts;      // [ws][kMaxChunks][L] int32: rows source s sent to local expert l up to the END of chunk c
    size_t off_flags;       // [kNumFlagKinds][A2A_MAX_WORLD][kFlagStride] u32 epochs, written by the peers
    size_t off_stage;       // [ws][T_max][stage_row_bytes]: one wire row per (source, token)   (DEDUP / FP8)
    // pipelined schedule only: what a source tells a destination about the wire rows it sends there
    size_t off_rec_tok;     // [ws][T_max] int32: token of wire row n of source s
    size_t off_rec_ent;     // [ws][T_max][K] u32: (local expert << 16 | slot) of pair k of that token, or kNoEntry
    size_t off_rec_w;       // [ws][T_max][K] f32: the token's top-k weights (used when the expert rank reduces)
    size_t off_hdr;         // [ws][8] int32: [0] = number of wire rows source s sent in this call
    size_t off_ret;         // [ws][T_max][H] elements: partial sums pushed home by expert rank d (PUSH combine)
    int stage_row_bytes;
    int senders;            // blocks of the pipelined kernel that only move rows to the peers
    int routers;            // router blocks per destination rank (each writes the records of a slice of the tokens)
    int rank, ws, E, K, H, T_max, L;
    int T;                  // tokens of this rank in the current call
    int chunks;             // token chunks per call, 1..kMaxChunks (same on every rank)
    int wpc;                // 32-token bitmap words per chunk: chunk c = tokens [32*c*wpc, 32*(c+1)*wpc)
    uint32_t epoch;
    long long timeout_ns;
    // local scratch of this rank
    int* slot;              // [T_max*K] slot of pair (t,k) inside slab (expert, this rank), -1 = dropped
    int* send_counts;       // [E]
    uint32_t* tickets;      // [2][kMaxChunks] block-arrival counters, one per publishing phase and chunk
    uint32_t* ptickets;     // [2][A2A_MAX_WORLD] pipelined schedule: arrivals per destination / per source
    uint32_t* seen;         // [2][A2A_MAX_WORLD][kFlagStride] local re-publication of the peers' dispatch / expert flags
    a2a_status_t* status;
    long long* trace;       // [blocks][kNumStamps] or nullptr when tracing is off
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

__device__ __forceinline__ void stamp(const DevParams& p, int which) {
    if (p.trace != nullptr && threadIdx.x == 0) {
        p.trace[(size_t)blockIdx.x * kNumStamps + which] = clock64();
        if (which == kStampStart) p.trace[(size_t)blockIdx.x * kNumStamps + kStampGlobalNs] = global_ns();
    }
}

// Stamp by whichever thread the caller elects (exactly one per block and slot).
__device__ __forceinline__ void stamp_by(const DevParams& p, int which, bool elected) {
    if (p.trace != nullptr && elected) p.trace[(size_t)blockIdx.x * kNumStamps + which] = clock64();
}

// Value stamp (not a time): e.g. the role of the block.
__device__ __forceinline__ void stamp_value(const DevParams& p, int which, long long v) {
    if (p.trace != nullptr && threadIdx.x == 0) p.trace[(size_t)blockIdx.x * kNumStamps + which] = v;
}

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Strong (L1-bypassing) load without ordering: what a spin loop polls with.  Polling with
// acquire loads would execute a fence per iteration in every waiting block.
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ uint32_t ld_relaxed_gpu(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ void fence_acq_rel_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }

__device__ __forceinline__ void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }

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

// Loads of data another GPU, another block or an earlier phase produced: skip L1.
__device__ __forceinline__ uint4 ld_stream(const uint4* p) { return __ldcg(p); }
__device__ __forceinline__ uint2 ld_stream(const uint2* p) { return __ldcg(p); }
__device__ __forceinline__ int ld_stream(const int* p) { return __ldcg(p); }
__device__ __forceinline__ float ld_stream(const float* p) { return __ldcg(p); }

// Stores that this SM will not read back.
__device__ __forceinline__ void st_stream(uint4* p, uint4 v) { __stcg(p, v); }
__device__ __forceinline__ void st_stream(uint2* p, uint2 v) { __stcg(p, v); }

// The status record in device memory, followed by the address of a word in mapped host memory
// that mirrors `code`: the host can see that something was recorded without any CUDA call.
struct StatusBlock {
    a2a_status_t s;
    int* host_code;
};

__device__ __forceinline__ void mirror_code(a2a_status_t* st, int code) {
    int* host = reinterpret_cast<StatusBlock*>(st)->host_code;
    if (host != nullptr) *reinterpret_cast<volatile int*>(host) = code;
}

__device__ __forceinline__ void record_error(a2a_status_t* st, int code, int rank, int peer, int phase,
                                             uint32_t epoch, int detail) {
    if (atomicCAS(&st->code, 0, code) == 0) {
        st->rank = rank;
        st->peer = peer;
        st->phase = phase;
        st->epoch = epoch;
        st->detail = detail;
        mirror_code(st, code);
        __threadfence();
    }
}

__device__ __forceinline__ uint32_t* flag_ptr(uint8_t* region_base, size_t off_flags, int kind, int index) {
    return reinterpret_cast<uint32_t*>(region_base + off_flags) + ((size_t)kind * A2A_MAX_WORLD + index) * kFlagStride;
}

__device__ __forceinline__ void record_timeout(const DevParams& p, int phase, int peer, uint32_t epoch) {
    // a timeout outranks whatever was recorded before: the other waiters key on it
    if (atomicExch(&p.status->code, A2A_ERR_TIMEOUT) != A2A_ERR_TIMEOUT) {
        p.status->rank = p.rank;
        p.status->peer = peer;
        p.status->phase = phase;
        p.status->epoch = epoch;
        p.status->detail = 0;
        mirror_code(p.status, A2A_ERR_TIMEOUT);
        __threadfence();
    }
}

// Spin until the epoch read through `load()` has reached `epoch` (wrap-safe), then run
// `acquire()` (the fence of the right scope).  Gives up after timeout_ns, or as soon as
// any thread of this rank has recorded a timeout (one missing peer costs one budget, not
// one per waiter), and returns false.
template <typename Load, typename Acquire>
__device__ __forceinline__ bool wait_epoch(Load load, Acquire acquire, uint32_t epoch, const DevParams& p, int phase,
                                           int peer) {
    long long t0 = 0;
    unsigned backoff = 32;
    for (int spins = 0;; ++spins) {
        if ((int32_t)(load() - epoch) >= 0) {
            acquire();  // relaxed load + fence = acquire
            return true;
        }
        if (spins == 0) {
            t0 = global_ns();
            continue;
        }
        if (ld_volatile_i32(&p.status->code) == A2A_ERR_TIMEOUT) return false;
        if (global_ns() - t0 > p.timeout_ns) {
            record_timeout(p, phase, peer, epoch);
            return false;
        }
        __nanosleep(backoff);
        if (backoff < 256) backoff <<= 1;
    }
}

// A flag another GPU writes: polled with strong system-scope loads; ONE system-scope acquire
// fence on success (only watcher threads and the barrier kernel come through here).
__device__ __forceinline__ bool wait_flag_sys(const uint32_t* flag, uint32_t epoch, const DevParams& p, int phase, int peer) {
    return wait_epoch([flag] { return ld_relaxed_sys(flag); }, [] { fence_acq_rel_sys(); }, epoch, p, phase, peer);
}

// A word a thread of this GPU writes: gpu scope.
__device__ __forceinline__ bool wait_flag_gpu(const uint32_t* flag, uint32_t epoch, const DevParams& p, int phase, int peer) {
    return wait_epoch([flag] { return ld_relaxed_gpu(flag); }, [] { fence_acq_rel_gpu(); }, epoch, p, phase, peer);
}

// What a flag word carries once chunk c of this call is published: monotonic over calls and chunks.
__device__ __forceinline__ uint32_t flag_value(const DevParams& p, int c) { return p.epoch * 8u + (uint32_t)c + 1u; }

// First and one-past-last token of chunk c.
__device__ __forceinline__ int chunk_begin(const DevParams& p, int c) { return min(p.T, 32 * c * p.wpc); }
__device__ __forceinline__ int chunk_end(const DevParams& p, int c) {
    return c == p.chunks - 1 ? p.T : min(p.T, 32 * (c + 1) * p.wpc);
}

__device__ __forceinline__ uint32_t* seen_ptr(const DevParams& p, int kind, int index) {
    return p.seen + ((size_t)kind * A2A_MAX_WORLD + index) * kFlagStride;
}

// Watcher duty: wait for peer `index`'s flag of `kind` at system scope, then hand it to
// the rest of this GPU through the local word.  On a timeout nothing is handed on and
// the local waiters run into the recorded timeout.
__device__ __forceinline__ void st_relaxed_gpu(uint32_t* p, uint32_t v) {
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ bool watch_and_republish(const DevParams& p, int kind, int index, int phase, uint32_t value) {
    const bool ok = wait_flag_sys(flag_ptr(p.peer[p.rank], p.off_flags, kind, index), value, p, phase, index);
    // the system-scope acquire-release fence taken on success also is the release half of this store
    // (a fence followed by a relaxed store releases at the fence's scope, which includes the gpu's)
    if (ok) st_relaxed_gpu(seen_ptr(p, kind, index), value);
    return ok;
}

// All threads of the block call this after their last store of a phase.  Returns true in
// exactly one block of the grid: the one that arrived last.  The caller of that block
// must fence (system scope) before it publishes; every store of every block is then
// ordered before the publication.
__device__ __forceinline__ bool grid_arrive_last(uint32_t* ticket) {
    __shared__ int s_last;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();  // gpu scope: cheap, and enough between blocks of one GPU
        const uint32_t t = atomicAdd(ticket, 1u);
        const int last = (t == gridDim.x - 1);
        if (last) *ticket = 0;  // everyone has arrived: re-arm for the next launch
        s_last = last;
    }
    __syncthreads();
    return s_last != 0;
}

// Exclusive prefix sum over n <= 4*kThreads ints held in shared memory `a`
// (in place; a[n] receives the total).  All kThreads threads must call it.
__device__ __forceinline__ void block_exclusive_scan(int* a, int n) {
    __shared__ int s_warp[kThreads / 32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int per = (n + kThreads - 1) / kThreads;
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
    if (tid == kThreads - 1) a[n] = base + inc;
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

// ---- bulk asynchronous copies (the copy engine of the SM) and their mbarriers ----------
// Only the plain forms are used: one CTA's shared memory, no cluster-wide delivery.
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

// Makes the initialised barriers visible to the copy engine.
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// global -> this CTA's shared memory; completion is counted in bytes on `bar`.
// dst, src and bytes must be multiples of 16.
__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

// this CTA's shared memory -> global (local or a peer's); joins the thread's current bulk group.
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src_smem, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }

// At most N of this thread's most recent bulk groups may still be READING shared memory.
template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }

// At most n (0..5; larger waits for 5) of this thread's most recent bulk groups may still be pending
// at all: the older ones have written their destination.
__device__ __forceinline__ void bulk_wait_done(int n) {
    switch (n) {
        case 0: asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); break;
        case 1: asm volatile("cp.async.bulk.wait_group 1;" ::: "memory"); break;
        case 2: asm volatile("cp.async.bulk.wait_group 2;" ::: "memory"); break;
        case 3: asm volatile("cp.async.bulk.wait_group 3;" ::: "memory"); break;
        case 4: asm volatile("cp.async.bulk.wait_group 4;" ::: "memory"); break;
        default: asm volatile("cp.async.bulk.wait_group 5;" ::: "memory"); break;
    }
}
constexpr int kArrivalLag = 4;  // stores a sender issues after a destination's last one before it waits for that one

// Orders the copy engine's accesses to global memory with this thread's ordinary ones.
__device__ __forceinline__ void fence_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }
// ... and its reads of shared memory after ordinary stores to it.
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

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

// The placeholder expert op on 8 elements: dtype(float(x) * scale), one rounding.
template <typename T>
__device__ __forceinline__ uint4 scale8(const uint4& v, float scale) {
    float f[8];
    unpack8<T>(v, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] *= scale;
    return pack8<T>(f);
}

// 8 floats -> 8 e4m3 bytes (round to nearest even, saturating to +-448)
__device__ __forceinline__ uint2 pack8_e4m3(const float (&f)[8]) {
    uint2 q;
    unsigned short h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
        h[i] = __nv_cvt_float2_to_fp8x2(make_float2(f[2 * i], f[2 * i + 1]), __NV_SATFINITE, __NV_E4M3);
    q.x = (unsigned)h[0] | ((unsigned)h[1] << 16);
    q.y = (unsigned)h[2] | ((unsigned)h[3] << 16);
    return q;
}

// 8 e4m3 bytes -> 8 floats (exact)
__device__ __forceinline__ void unpack8_e4m3(const uint2& q, float (&f)[8]) {
    const unsigned short h[4] = {(unsigned short)(q.x & 0xffff), (unsigned short)(q.x >> 16),
                                 (unsigned short)(q.y & 0xffff), (unsigned short)(q.y >> 16)};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __half2_raw r = __nv_cvt_fp8x2_to_halfraw2(h[i], __NV_E4M3);
        const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&r));
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}

}  // namespace a2a
