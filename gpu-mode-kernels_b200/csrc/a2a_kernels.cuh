// The hot path: routing, dispatch (send / receive), expert placeholder, combine --
// as phases (device functions) that run either as separate kernels (the public
// phase entry points) or back to back inside ONE cooperative kernel (a2a_forward).
// Hand-written for sm_100a.  Every phase is bound by NVLink or HBM bandwidth (there
// is no contraction on this path), so the work is 16-byte vector traffic spread over
// a grid that is a multiple of the SM count, with as few system-scope fences as possible.
#pragma once

#include "a2a_device.cuh"

namespace a2a {

// ---------------------------------------------------------------------------
// Shared-memory carve-up of a block (dynamic shared memory, ints):
//   bits [Wc][E]  bit t%32 of word t/32 set iff token t of this rank uses expert e
//   wpre [Wc][E]  number of set bits in the words before w (exclusive scan over w)
//   cnt  [E]      tokens using expert e = rows this rank sends to e
//   pre  [E+2]    receive side: prefix sums over the slabs of a source
//   base [E]      receive side: first slot of the current chunk in every slab of a source
//   idx  [T*K]    this rank's top-k expert indices (one coalesced pass over global memory;
//                 every later look-up, including the repeat check, is a shared-memory read)
// Wc = ceil(T/32) words of the current call; the allocation is sized for T_max.
// ---------------------------------------------------------------------------
struct BlockSmem {
    unsigned* bits;
    int* wpre;
    int* cnt;
    int* pre;
    int* base;
    int* idx;
};

__host__ __device__ inline size_t pre_ints(int E, int /*T_max*/) { return (size_t)E + 2; }

__host__ __device__ inline size_t block_smem_ints(int E, int T_max, int K) {
    const size_t W = (size_t)(T_max + 31) / 32;
    return 2 * W * E + E + pre_ints(E, T_max) + E + (size_t)T_max * K;
}

__device__ __forceinline__ BlockSmem carve_smem(int* base, int E, int T_max) {
    const size_t W = (size_t)(T_max + 31) / 32;
    BlockSmem s;
    s.bits = reinterpret_cast<unsigned*>(base);
    s.wpre = base + W * E;
    s.cnt = base + 2 * W * E;
    s.pre = s.cnt + E;
    s.base = s.pre + pre_ints(E, T_max);
    s.idx = s.base + E;
    return s;
}

// ---------------------------------------------------------------------------
// Routing.  Top-k experts of one token are distinct, so the slot of pair (t,k)
// inside slab (expert e, this source) -- "number of earlier pairs of this rank
// with the same expert", the order of the CPU reference (reference.py:79-86,
// :140-146) -- equals the number of tokens t' < t that use e.  Every block builds
// the [expert x token] bitmap of the whole rank in its own shared memory (T*K
// atomicOr on shared memory, 8 KB of indices from L2), scans the words per expert,
// and can then answer any slot with one popc.  A pair whose expert is out of range,
// or repeats an expert of an earlier k of its token, is reported (A2A_ERR_ROUTING)
// and dropped: it gets slot -1, sends nothing and contributes nothing.
// ---------------------------------------------------------------------------
__device__ __forceinline__ bool pair_is_valid(const DevParams& p, const BlockSmem& s, int t, int k, int e) {
    if (e < 0 || e >= p.E) return false;
    const int* row = s.idx + t * p.K;
    bool repeat = false;
    for (int kk = 0; kk < k; ++kk) repeat |= (row[kk] == e);
    return !repeat;
}

__device__ __forceinline__ void route_build(const DevParams& p, const BlockSmem& s) {
    const int tid = threadIdx.x;
    const int E = p.E, K = p.K, P = p.T * p.K;
    const int Wc = (p.T + 31) >> 5;
    for (int pair = tid; pair < P; pair += kThreads) s.idx[pair] = __ldg(p.idx + pair);
    for (int i = tid; i < Wc * E; i += kThreads) s.bits[i] = 0u;
    __syncthreads();
    // one token per thread: no division, K consecutive indices (one or two 32-byte sectors)
    for (int t = tid; t < p.T; t += kThreads) {
        const int* row = p.idx + (size_t)t * K;
        const unsigned bit = 1u << (t & 31);
        unsigned* word = s.bits + (t >> 5) * E;
        for (int k = 0; k < K; ++k) {
            const int e = __ldg(row + k);
            if (e < 0 || e >= E) {
                record_error(p.status, A2A_ERR_ROUTING, p.rank, -1, kPhaseRoute, p.epoch, e);
            } else if (atomicOr(word + e, bit) & bit) {  // only this thread sets this bit: a repeat inside the token
                record_error(p.status, A2A_ERR_ROUTING, p.rank, -1, kPhaseRoute, p.epoch, e);
            }
        }
    }
    __syncthreads();
    for (int e = tid; e < E; e += kThreads) {
        int run = 0;
        for (int w = 0; w < Wc; ++w) {
            s.wpre[w * E + e] = run;
            run += __popc(s.bits[w * E + e]);
        }
        s.cnt[e] = run;
    }
    __syncthreads();
}

// Slot of pair (t,k) with expert e, or -1 if the pair is dropped.
__device__ __forceinline__ int pair_slot(const DevParams& p, const BlockSmem& s, int t, int k, int e) {
    if (!pair_is_valid(p, s, t, k, e)) return -1;
    const int w = t >> 5;
    return s.wpre[w * p.E + e] + __popc(s.bits[w * p.E + e] & ((1u << (t & 31)) - 1u));
}

// Publication of one chunk of a phase by all threads of the block that arrived last.  Our
// own rank is served first and at gpu scope (its consumers are blocks of this GPU); the
// peers get ONE system fence, then the chunk's flag value in their flag word of `kind`.
__device__ __forceinline__ void publish_flags(const DevParams& p, int kind, uint32_t value) {
    const int tid = threadIdx.x;
    __syncthreads();  // whatever the block wrote for this publication has been issued
    if (tid == 0) st_release_gpu(seen_ptr(p, kind, p.rank), value);  // fence.gpu + store
    if (p.ws > 1) {
        if (tid == 0) __threadfence_system();  // orders every block's rows (seen through the tickets) for the peers
        __syncthreads();
        if (tid < p.ws && tid != p.rank) st_relaxed_sys(flag_ptr(p.peer[tid], p.off_flags, kind, p.rank), value);
    }
}

// Rows this rank sends to expert e from the tokens before the end of chunk c.
__device__ __forceinline__ int sent_up_to_chunk(const DevParams& p, const BlockSmem& s, int c, int e) {
    const int Wc = (p.T + 31) >> 5;
    const int wb = (c + 1) * p.wpc;
    return (c == p.chunks - 1 || wb >= Wc) ? s.cnt[e] : s.wpre[wb * p.E + e];
}

// Dispatch publication of chunk c.  Routing is known before any row moves, so the first
// chunk carries the cumulative row counts of EVERY chunk for every (this source, local
// expert) slab; later chunks only raise the flag.
__device__ __forceinline__ void publish_dispatch(const DevParams& p, const BlockSmem& s, int c) {
    if (c == 0) {
        for (int i = threadIdx.x; i < p.E * p.chunks; i += kThreads) {
            const int cc = i / p.E, e = i - cc * p.E;
            const int d = e / p.L, l = e - d * p.L;
            reinterpret_cast<int*>(p.peer[d] + p.off_counts)[((size_t)p.rank * kMaxChunks + cc) * p.L + l] =
                sent_up_to_chunk(p, s, cc, e);
        }
        for (int e = threadIdx.x; e < p.E; e += kThreads) p.send_counts[e] = s.cnt[e];
    }
    publish_flags(p, kFlagDispatch, flag_value(p, c));
}

// Copy one row of nvec 16-byte vectors with all 256 threads, up to four loads in flight each.
__device__ __forceinline__ void copy_row(const uint4* __restrict__ src, uint4* __restrict__ dst, int nvec) {
    const int tid = threadIdx.x;
    for (int v0 = 0; v0 < nvec; v0 += kThreads * 4) {
        uint4 r[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int v = v0 + u * kThreads + tid;
            if (v < nvec) r[u] = ld_input(src + v);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int v = v0 + u * kThreads + tid;
            if (v < nvec) st_stream(dst + v, r[u]);
        }
    }
}

// ---------------------------------------------------------------------------
// Dispatch, sending half.  Never waits.
// DIRECT: one block per (token, k) pair at a time; the row goes straight into slab
//   (expert, this rank) on the expert's rank (NVLink for a peer, HBM for ourselves).
// DEDUP / FP8: one block per (token, destination rank); the row crosses the wire
//   once per destination into stage[src][t] (FP8: quantised on the fly, one fp32
//   scale per 128 values); every slab row that wants it gets its (token, k) word,
//   through which the receiver finds the wire row when it fans out.
// Work is done chunk of tokens by chunk; the block that finishes a chunk last publishes it.
// ---------------------------------------------------------------------------
template <typename T, int PAYLOAD>
__device__ __forceinline__ void send_chunk(const DevParams& p, const BlockSmem& s, int c) {
    const int tid = threadIdx.x;
    const int K = p.K, nvec = p.H >> 3;
    const int ta = chunk_begin(p, c), tb = chunk_end(p, c);  // this chunk's tokens
    if (PAYLOAD == A2A_PAYLOAD_DIRECT) {
        for (int pair = ta * K + (int)blockIdx.x; pair < tb * K; pair += gridDim.x) {
            const int t = pair / K, k = pair - t * K;
            const int e = s.idx[pair];
            const int j = pair_slot(p, s, t, k, e);
            if (tid == 0) p.slot[pair] = j;
            if (j < 0) continue;
            const int d = e / p.L, l = e - d * p.L;
            const size_t row = ((size_t)l * p.ws + p.rank) * p.T_max + j;
            copy_row(reinterpret_cast<const uint4*>(p.x) + (size_t)t * nvec,
                     reinterpret_cast<uint4*>(p.peer[d] + p.off_rows) + row * nvec, nvec);
            if (tid == 0) reinterpret_cast<int*>(p.peer[d] + p.off_meta)[row] = (t << 8) | k;
        }
    } else {
        for (int it = ta * p.ws + (int)blockIdx.x; it < tb * p.ws; it += gridDim.x) {
            const int t = it / p.ws, d = it - t * p.ws;
            // which of the token's experts live on d: each of them gets its slab row's (token, k)
            // word there; the row itself crosses the wire once
            int hit = 0;
            if (tid < K) {
                const int e = s.idx[t * K + tid];
                const bool in_range = (e >= 0 && e < p.E);
                const int home = in_range ? e / p.L : 0;  // an out-of-range pair is booked (as dropped) by item d = 0
                if (home == d) {
                    const int j = pair_slot(p, s, t, tid, e);
                    p.slot[(size_t)t * K + tid] = j;
                    if (j >= 0) {
                        const size_t row = ((size_t)(e - d * p.L) * p.ws + p.rank) * p.T_max + j;
                        reinterpret_cast<int*>(p.peer[d] + p.off_meta)[row] = (t << 8) | tid;
                        hit = 1;
                    }
                }
            }
            if (!__syncthreads_or(hit)) continue;  // nothing of this token lives on d
            uint8_t* wire = p.peer[d] + p.off_stage + ((size_t)p.rank * p.T_max + t) * p.stage_row_bytes;
            const uint4* src = reinterpret_cast<const uint4*>(p.x) + (size_t)t * nvec;
            if (PAYLOAD == A2A_PAYLOAD_DEDUP) {
                copy_row(src, reinterpret_cast<uint4*>(wire), nvec);
            } else {
                // nvec is a multiple of 16 (H % 128 == 0): the 16 lanes of a scale block are all in or all out
                for (int v0 = 0; v0 < nvec; v0 += kThreads) {
                    const int v = v0 + tid;
                    float f[8];
                    float amax = 0.f;
                    if (v < nvec) {
                        unpack8<T>(ld_input(src + v), f);
#pragma unroll
                        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
                    }
#pragma unroll
                    for (int o = 8; o >= 1; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
                    if (v < nvec) {
                        const float scale = amax > 0.f ? amax / 448.f : 1.f;
#pragma unroll
                        for (int i = 0; i < 8; ++i) f[i] = f[i] / scale;
                        st_stream(reinterpret_cast<uint2*>(wire) + v, pack8_e4m3(f));
                        if ((v & 15) == 0) reinterpret_cast<float*>(wire + p.H)[v >> 4] = scale;
                    }
                }
            }
        }
    }
    if (grid_arrive_last(p.tickets + kTicketSend * kMaxChunks + c)) publish_dispatch(p, s, c);
}

// The sending half as its own kernel: routing, then every chunk in order.
template <typename T, int PAYLOAD>
__device__ __forceinline__ void send_phase(const DevParams& p, const BlockSmem& s) {
    stamp(p, kStampStart);
    route_build(p, s);
    stamp(p, kStampRouted);
    for (int c = 0; c < p.chunks; ++c) send_chunk<T, PAYLOAD>(p, s, c);
    stamp(p, kStampSent);
}

// ---------------------------------------------------------------------------
// Receive side.  Blocks are partitioned over the source ranks (block b serves source
// b % ws), so the rows of a source are processed as soon as THAT source's flag has
// arrived.  The first block of every source is its watcher (system scope); the others
// wait on the local word.  Template switches:
//   WAIT    wait (bounded) for the source's dispatch flag of this call
//   FANOUT  DEDUP/FP8 payloads: fill every valid slab row from the wire row of its token
//           (FP8: dequantise to T first)
//   SCALE   the placeholder expert op on the valid slab rows: in place, or with FANOUT
//           applied while fanning out
//   PUBLISH tell every home rank that this rank's expert outputs are ready
// ---------------------------------------------------------------------------
// The valid rows of source s, flattened over the local experts with a prefix sum of the
// counts so that skewed routing does not idle blocks; one block per row at a time.
//   FANOUT (staged payloads): the row's content comes from the wire row of its token
//          (found through the row's (token, k) word), FP8: dequantised and rounded to T;
//   SCALE: the placeholder expert op, T(float(row) * (1 + rank)), on the way.
// Without FANOUT the row is read from the slab itself (in place).
template <typename T, int PAYLOAD, bool FANOUT, bool SCALE>
__device__ __forceinline__ void rows_of_source(const DevParams& p, int* pre, int* base, int s, int c, int part,
                                               int nparts) {
    constexpr bool from_wire = FANOUT && PAYLOAD != A2A_PAYLOAD_DIRECT;
    constexpr bool fp8 = from_wire && PAYLOAD == A2A_PAYLOAD_FP8;
    const int tid = threadIdx.x;
    uint8_t* self = p.peer[p.rank];
    // rows of chunk c in slab (l, s): slots [counts up to chunk c-1, counts up to chunk c)
    const int* counts = reinterpret_cast<const int*>(self + p.off_counts) + ((size_t)s * kMaxChunks + c) * p.L;
    for (int l = tid; l < p.L; l += kThreads) {
        int hi = ld_stream(counts + l);
        int lo = c > 0 ? ld_stream(counts - p.L + l) : 0;
        if (lo < 0 || hi < lo || hi > p.T_max) {
            record_error(p.status, A2A_ERR_CAPACITY, p.rank, s, kPhaseExpert, p.epoch, hi);
            lo = hi = 0;
        }
        pre[l] = hi - lo;
        base[l] = lo;
    }
    block_exclusive_scan(pre, p.L);
    const int total = pre[p.L];
    const int nvec = p.H >> 3;
    const float scale = (float)(1 + p.rank);
    uint4* rows = reinterpret_cast<uint4*>(self + p.off_rows);
    const int* meta = reinterpret_cast<const int*>(self + p.off_meta);
    for (int r = part; r < total; r += nparts) {
        const int l = upper_slab(pre, p.L, r);
        const int j = base[l] + r - pre[l];
        const size_t ri = ((size_t)l * p.ws + s) * p.T_max + j;
        uint4* row = rows + ri * nvec;
        const uint8_t* wire = nullptr;
        if (from_wire) {
            int t = ld_stream(meta + ri) >> 8;
            if (t < 0 || t >= p.T_max) {
                record_error(p.status, A2A_ERR_CAPACITY, p.rank, s, kPhaseRecv, p.epoch, t);
                continue;
            }
            wire = self + p.off_stage + ((size_t)s * p.T_max + t) * p.stage_row_bytes;
        }
        for (int v0 = 0; v0 < nvec; v0 += kThreads * 4) {
            uint4 q[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int v = v0 + u * kThreads + tid;
                if (v < nvec) {
                    if (fp8) {
                        float f[8];
                        unpack8_e4m3(ld_stream(reinterpret_cast<const uint2*>(wire) + v), f);
                        const float sc = ld_stream(reinterpret_cast<const float*>(wire + p.H) + (v >> 4));
#pragma unroll
                        for (int i = 0; i < 8; ++i) f[i] *= sc;
                        q[u] = pack8<T>(f);  // the received row, rounded to T as the receiver stores it
                    } else if (from_wire) {
                        q[u] = ld_stream(reinterpret_cast<const uint4*>(wire) + v);
                    } else {
                        q[u] = ld_stream(row + v);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int v = v0 + u * kThreads + tid;
                if (v < nvec) st_stream(row + v, SCALE ? scale8<T>(q[u], scale) : q[u]);
            }
        }
    }
}

template <typename T, int PAYLOAD, bool WAIT, bool FANOUT, bool SCALE, bool PUBLISH>
__device__ __forceinline__ void expert_chunk(const DevParams& p, const BlockSmem& sm, int c) {
    __shared__ int s_seen;
    const int tid = threadIdx.x;
    const uint32_t want = flag_value(p, c);
    // block b serves source b % ws together with the other blocks of that residue;
    // a grid smaller than the world size lets each block walk several sources alone
    const bool many = (int)gridDim.x >= p.ws;
    const int s_first = many ? (int)blockIdx.x % p.ws : (int)blockIdx.x;
    const int s_step = many ? p.ws * A2A_MAX_WORLD : (int)gridDim.x;  // many: exactly one source
    for (int s = s_first; s < p.ws; s += s_step) {
        const int part = many ? (int)blockIdx.x / p.ws : 0;
        const int nparts = many ? ((int)gridDim.x - s + p.ws - 1) / p.ws : 1;
        if (WAIT) {
            // part 0 watches a peer's flag at system scope and hands it on; the rest, and everybody
            // for our own rank (whose publisher writes the local word itself), wait locally
            if (tid == 0)
                s_seen = (part == 0 && s != p.rank
                              ? watch_and_republish(p, kFlagDispatch, s, kPhaseRecv, want)
                              : wait_flag_gpu(seen_ptr(p, kFlagDispatch, s), want, p, kPhaseRecv, s)) ? 1 : 0;
            __syncthreads();
            const int seen = s_seen;
            __syncthreads();
            if (!seen) break;  // timeout recorded; the rows of this source are left alone
            if (c == 0) stamp(p, kStampDispatchSeen);
        }
        constexpr bool staged = (PAYLOAD != A2A_PAYLOAD_DIRECT);
        if ((staged && FANOUT) || SCALE)
            rows_of_source<T, PAYLOAD, FANOUT, SCALE>(p, sm.pre, sm.base, s, c, part, nparts);
        __syncthreads();  // sm.pre / sm.base are reused by the next source
    }
    if (PUBLISH) {
        if (grid_arrive_last(p.tickets + kTicketExpert * kMaxChunks + c)) {
            // after a timeout the outputs are incomplete: say nothing, the home ranks run into their own budget
            if (tid == 0) s_seen = (ld_volatile_i32(&p.status->code) != A2A_ERR_TIMEOUT) ? 1 : 0;
            __syncthreads();
            if (s_seen) publish_flags(p, kFlagExpert, want);
        }
    }
}

// The receive side as its own kernel: every chunk in order.
template <typename T, int PAYLOAD, bool WAIT, bool FANOUT, bool SCALE, bool PUBLISH>
__device__ __forceinline__ void expert_phase(const DevParams& p, const BlockSmem& sm) {
    for (int c = 0; c < p.chunks; ++c) expert_chunk<T, PAYLOAD, WAIT, FANOUT, SCALE, PUBLISH>(p, sm, c);
    stamp(p, kStampExpertDone);
}

// ---------------------------------------------------------------------------
// Combine (pull).  A warp owns 64 consecutive 16-byte vectors (1 KB) of one
// token's output.  Lane k < K looks up pair (t,k): expert, slot (known from routing,
// so no metadata is fetched), weight, and waits (bounded) until the expert's rank has
// published its outputs -- warp d of the grid is the watcher of rank d's flag, the
// others wait on the local word; only then is the pair's slot read.  Pointer and weight are then broadcast by shuffles and
// every lane pulls its two 16-byte vectors of each of the K rows from the rank that holds
// them, sixteen loads in flight, accumulating float(row) * w in fp32 in k order.
// ---------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void combine_phase(const DevParams& p, int cb, int ncb, bool own_watchers) {
    const int lane = threadIdx.x & 31;
    const int warp = cb * (kThreads / 32) + (threadIdx.x >> 5);
    const int nwarps = ncb * (kThreads / 32);
    const int K = p.K, nvec = p.H >> 3;
    const int nseg = (nvec + 63) >> 6;  // a warp owns 64 consecutive vectors (1 KB) of one token's output
    for (int c = 0; c < p.chunks; ++c) {
    const uint32_t want = flag_value(p, c);
    const int ta = chunk_begin(p, c), tb = chunk_end(p, c);
    const int items = (tb - ta) * nseg;
    // warp d of the grid watches rank d's flag for this chunk before its own items (unless the
    // caller has watchers of its own)
    if (own_watchers && warp < p.ws && warp != p.rank && lane == 0)
        watch_and_republish(p, kFlagExpert, warp, kPhaseCombine, want);
    __syncwarp();
    unsigned ready = 0u;  // ranks this lane has already seen ready for this chunk
    for (int item = warp; item < items; item += nwarps) {
        const int t = ta + item / nseg, seg = item % nseg;
        const int v0 = seg * 64 + lane, v1 = v0 + 32;
        unsigned long long my_row = 0ull;
        float my_w = 0.f;
        bool ok = true;
        if (lane < K) {
            const size_t pair = (size_t)t * K + lane;
            const int e = __ldg(p.idx + pair);
            if (e >= 0 && e < p.E) {
                // The expert's rank is known from the caller's indices alone.  Its flag is awaited BEFORE
                // the slot table is read: the flag implies that this rank's own routing of this call (which
                // other blocks of this grid may still be writing) was complete when the rows left.
                const int d = e / p.L, l = e - d * p.L;
                if (!((ready >> d) & 1u)) {
                    ok = wait_flag_gpu(seen_ptr(p, kFlagExpert, d), want, p, kPhaseCombine, d);
                    ready |= 1u << d;
                }
                const int j = ok ? ld_stream(p.slot + pair) : -1;
                if (j >= 0) {
                    my_w = __ldg(p.w + pair);
                    my_row = reinterpret_cast<unsigned long long>(
                        reinterpret_cast<const uint4*>(p.peer[d] + p.off_rows) +
                        (((size_t)l * p.ws + p.rank) * p.T_max + j) * nvec);
                }
            }
        }
        if (!__all_sync(0xffffffffu, ok)) return;  // timeout recorded; leave the remaining output untouched
        if (item == warp && c == 0) stamp(p, kStampExpertSeen);
        float acc[2][8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[0][i] = acc[1][i] = 0.f;
        // eight rows at a time, two 16-byte vectors of each per lane: sixteen loads are on their way over
        // NVLink before the first is used (a pull is a round trip; what counts is how much is in flight)
        for (int k0 = 0; k0 < K; k0 += 8) {
            uint4 q[8][2];
            float w[8];
            bool have[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int k = (k0 + u < K) ? k0 + u : 0;
                const unsigned long long row = __shfl_sync(0xffffffffu, my_row, k);
                w[u] = __shfl_sync(0xffffffffu, my_w, k);
                have[u] = (k0 + u < K) && row != 0ull;
                if (have[u] && v0 < nvec) q[u][0] = ld_stream(reinterpret_cast<const uint4*>(row) + v0);
                if (have[u] && v1 < nvec) q[u][1] = ld_stream(reinterpret_cast<const uint4*>(row) + v1);
            }
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (have[u]) {
                    float f[8];
                    if (v0 < nvec) {
                        unpack8<T>(q[u][0], f);
#pragma unroll
                        for (int i = 0; i < 8; ++i) acc[0][i] = fmaf(f[i], w[u], acc[0][i]);
                    }
                    if (v1 < nvec) {
                        unpack8<T>(q[u][1], f);
#pragma unroll
                        for (int i = 0; i < 8; ++i) acc[1][i] = fmaf(f[i], w[u], acc[1][i]);
                    }
                }
        }
        if (v0 < nvec) st_stream(reinterpret_cast<uint4*>(p.y) + (size_t)t * nvec + v0, pack8<T>(acc[0]));
        if (v1 < nvec) st_stream(reinterpret_cast<uint4*>(p.y) + (size_t)t * nvec + v1, pack8<T>(acc[1]));
    }
    }  // chunks
    __syncthreads();
    stamp(p, kStampCombineDone);
}

// ---------------------------------------------------------------------------
// Kernels
// ---------------------------------------------------------------------------
extern __shared__ int a2a_dyn_smem[];

// Standalone routing: the slot table and send counts in global memory (what
// a2a_route promises); the sending kernel recomputes the same values in shared memory.
__global__ void __launch_bounds__(kThreads) route_kernel(const __grid_constant__ DevParams p) {
    const BlockSmem s = carve_smem(a2a_dyn_smem, p.E, p.T_max);
    route_build(p, s);
    const int P = p.T * p.K;
    for (int pair = threadIdx.x; pair < P; pair += kThreads) {
        const int t = pair / p.K, k = pair - t * p.K;
        p.slot[pair] = pair_slot(p, s, t, k, s.idx[pair]);
    }
    for (int e = threadIdx.x; e < p.E; e += kThreads) p.send_counts[e] = s.cnt[e];
}

template <typename T, int PAYLOAD>
__global__ void __launch_bounds__(kThreads) send_kernel(const __grid_constant__ DevParams p) {
    send_phase<T, PAYLOAD>(p, carve_smem(a2a_dyn_smem, p.E, p.T_max));
}

template <typename T, int PAYLOAD, bool WAIT, bool FANOUT, bool SCALE, bool PUBLISH>
__global__ void __launch_bounds__(kThreads) expert_kernel(const __grid_constant__ DevParams p) {
    expert_phase<T, PAYLOAD, WAIT, FANOUT, SCALE, PUBLISH>(p, carve_smem(a2a_dyn_smem, p.E, p.T_max));
}

template <typename T>
__global__ void __launch_bounds__(kThreads) combine_kernel(const __grid_constant__ DevParams p) {
    combine_phase<T>(p, (int)blockIdx.x, (int)gridDim.x, true);
}

// The whole path in one launch.  Launched cooperatively so that every block is
// resident: a block waits (bounded) on words that the last-finishing block of this very
// grid, or a peer GPU, will set.  The call is pipelined in token chunks: a block sends
// chunk c, then does its share of the expert work of chunk c-1 (whose rows had a whole
// chunk of sending time to land), so the phase boundaries of all but the last chunk hide
// behind NVLink-bound sending; the combine then walks the chunks in the same order.
// Publishing a chunk never depends on any receive-side work, so there is no wait cycle.
template <typename T, int PAYLOAD>
__global__ void __launch_bounds__(kThreads) forward_kernel(const __grid_constant__ DevParams p) {
    const BlockSmem s = carve_smem(a2a_dyn_smem, p.E, p.T_max);
    stamp(p, kStampStart);
    route_build(p, s);
    stamp(p, kStampRouted);
    for (int c = 0; c < p.chunks; ++c) {
        send_chunk<T, PAYLOAD>(p, s, c);
        if (c >= 1) expert_chunk<T, PAYLOAD, true, true, true, true>(p, s, c - 1);
    }
    stamp(p, kStampSent);
    expert_chunk<T, PAYLOAD, true, true, true, true>(p, s, p.chunks - 1);
    stamp(p, kStampExpertDone);
    combine_phase<T>(p, (int)blockIdx.x, (int)gridDim.x, true);
}

// ---------------------------------------------------------------------------
// Export: the reference's dispatch return value (reference.py:148) packed from the
// slabs -- rows of one expert ordered by (source rank, token, k).  Test helper.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) export_dispatch_kernel(const __grid_constant__ DevParams p, int* out_counts,
                                                                  uint4* out_rows, int* out_meta) {
    __shared__ int prefix[A2A_MAX_EXPERTS + 1];
    const int tid = threadIdx.x;
    uint8_t* self = p.peer[p.rank];
    const int nslab = p.L * p.ws;  // slab i = l * ws + s
    const int* counts = reinterpret_cast<const int*>(self + p.off_counts);
    for (int i = tid; i < nslab; i += kThreads) {
        const int l = i / p.ws, s = i - l * p.ws;
        const int c = counts[((size_t)s * kMaxChunks + p.chunks - 1) * p.L + l];
        prefix[i] = (c < 0 || c > p.T_max) ? 0 : c;
    }
    block_exclusive_scan(prefix, nslab);
    if (blockIdx.x == 0)
        for (int l = tid; l < p.L; l += kThreads) out_counts[l] = prefix[(l + 1) * p.ws] - prefix[l * p.ws];
    const int total = prefix[nslab];
    const int nvec = p.H >> 3;
    const size_t max_recv = (size_t)p.T_max * p.ws;
    const uint4* rows = reinterpret_cast<const uint4*>(self + p.off_rows);
    const int* meta = reinterpret_cast<const int*>(self + p.off_meta);
    for (int r = blockIdx.x; r < total; r += gridDim.x) {
        const int i = upper_slab(prefix, nslab, r);
        const int j = r - prefix[i];
        const int l = i / p.ws, s = i - l * p.ws;
        const size_t in_row = (size_t)i * p.T_max + j;
        const size_t out_row = (size_t)l * max_recv + (prefix[i] - prefix[l * p.ws]) + j;
        for (int v = tid; v < nvec; v += kThreads) out_rows[out_row * nvec + v] = rows[in_row * nvec + v];
        if (tid == 0) {
            const int m = meta[in_row];
            int* o = out_meta + out_row * 5;
            o[0] = p.rank * p.L + l;
            o[1] = s;
            o[2] = m >> 8;
            o[3] = m & 0xff;
            o[4] = 0;
        }
    }
}

// Cross-GPU rendezvous: announce to every peer, then wait for every peer (bounded).
__global__ void barrier_kernel(const __grid_constant__ DevParams p, uint32_t barrier_epoch) {
    const int tid = threadIdx.x;
    if (tid < p.ws) {
        __threadfence_system();
        st_release_sys(flag_ptr(p.peer[tid], p.off_flags, kFlagBarrier, p.rank), barrier_epoch);
        wait_flag_sys(flag_ptr(p.peer[p.rank], p.off_flags, kFlagBarrier, tid), barrier_epoch, p, kPhaseBarrier, tid);
    }
}

}  // namespace a2a
