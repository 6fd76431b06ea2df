// The pipelined schedule: the whole path in ONE cooperative launch whose blocks have
// fixed roles that run concurrently, so the NVLink transfers of dispatch and combine, the
// expert pass and the routing tables overlap instead of following each other.
//
//   senders  (p.senders blocks; one thread each drives the SM's copy engine)
//            For destination rank d = rank+1, rank+2, ... (a ring: at any moment every
//            rank sends to a different peer) the token rows wanted by d are bulk-loaded
//            from HBM into a six-stage shared-memory ring and bulk-stored straight into
//            d's stage buffer, one wire row per (token, destination).  No routing table is
//            needed for that, so rows move from the first microsecond.  When a
//            destination's last store has completed the block draws a ticket; the last
//            ticket (all senders + that destination's router) publishes the dispatch flag.
//   routers  (a few blocks per destination, then they join the experts)
//            build the [token x expert] bitmap of the destination's experts only, derive
//            the slot of every (token, k) row by popc, and write the destination its
//            records: per wire row the token, the (local expert, slot) of each pair and the
//            token's weights; plus per-slab counts and the (token, k) word of every slab row.
//   experts  (all other blocks) take the sources in arrival order (own rank first, then
//            rank-1, rank-2, ...).  Per wire row: read it once, write each slab row it
//            stands for (the dispatch output) with the placeholder expert op applied, and
//            -- PUSH combine -- accumulate w[t,k] * row in fp32 and return ONE partial row
//            per (token, this rank) to the home rank's return buffer over NVLink (packed in
//            shared memory and bulk-stored, like the senders' rows).  Inside a block warp 0
//            polls the sources' flags, warps 2-7 work, warp 1 draws the block's ticket per
//            source; the last ticket publishes the expert flag to that source.
//   watchers (spare warps of sender blocks 0 and 1) poll the peers' flags at system scope
//            and hand them to the rest of the GPU through local words.
//   combine  (every block, once its role is done) PUSH: y[t] = sum over the ranks that hold
//            experts of t of their partial rows, read from local memory.  PULL: each
//            (token, k) row is pulled from the expert's slab over NVLink and reduced with
//            the token's weights at home (the phase-by-phase combine, started per peer).
//
// Nothing here waits on work of its own role on another GPU, senders and routers never wait
// at all, and every wait is bounded; see a2a_device.cuh for the flag protocol.
#pragma once

#include "a2a_kernels.cuh"

namespace a2a {

enum PipeTicket : int { kPipeTicketDest = 0, kPipeTicketSource = 1 };

// ---- shared memory of a block, carved per role --------------------------------------------
// sender: ring [kStages][kStageBytes] | mbarriers [kStages] u64 | descriptors | list [ws][per] u16 | warp totals
// router: bits [Wc][L] | wpre [Wc][L] | cnt [L] | warp totals | wire row of each token of a round
__host__ __device__ inline int pipe_list_per(int T_max, int senders) { return (T_max + senders - 1) / (senders > 0 ? senders : 1); }

__host__ __device__ inline size_t pipe_sender_smem(int T_max, int ws, int senders) {
    size_t b = (size_t)kStages * kStageBytes + 128;                       // ring + barriers
    b += (size_t)kStages * 32;                                            // descriptors
    b += ((size_t)ws * pipe_list_per(T_max, senders) * 2 + 15) / 16 * 16; // token lists
    b += 8 * A2A_MAX_WORLD * 4;                                           // warp totals
    return b;
}

__host__ __device__ inline size_t pipe_router_smem(int T_max, int L) {
    const size_t W = (size_t)(T_max + 31) / 32;
    return (2 * W * L + L + 16 + 256) * 4;  // bitmap, prefix, counts, warp totals, wire row of a round's tokens
}

struct SendDesc {
    unsigned long long dst;  // destination address of the piece
    unsigned bytes;
    int dest_done;           // >= 0: this piece is the block's last one for that destination rank
};

// Ranks whose experts token t uses (in-range pairs only; a repeated expert adds no new rank).
__device__ __forceinline__ unsigned dest_mask(const DevParams& p, int t) {
    unsigned m = 0;
    const int* row = p.idx + (size_t)t * p.K;
    if ((p.K & 3) == 0 && (reinterpret_cast<uintptr_t>(p.idx) & 15) == 0) {  // the row is 16-byte aligned: vector loads
        for (int k = 0; k < p.K; k += 4) {
            const int4 e4 = __ldg(reinterpret_cast<const int4*>(row + k));
            const int e[4] = {e4.x, e4.y, e4.z, e4.w};
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (e[u] >= 0 && e[u] < p.E) m |= 1u << (e[u] / p.L);
        }
        return m;
    }
    for (int k = 0; k < p.K; ++k) {
        const int e = __ldg(row + k);
        if (e >= 0 && e < p.E) m |= 1u << (e / p.L);
    }
    return m;
}

// One arrival of a sender thread or a router block on destination d's ticket; the last of
// the `expected` arrivals publishes this rank's dispatch flag on d (for d = this rank: the
// local word the expert blocks wait on; only the routers arrive there).  Called by ONE thread
// whose own stores (and, through a barrier, its block's) are complete.
__device__ __forceinline__ void arrive_dest(const DevParams& p, int d, uint32_t expected) {
    fence_async_global();  // bulk stores of this thread, completed above, before the ordinary fence
    __threadfence();
    uint32_t* ticket = p.ptickets + kPipeTicketDest * A2A_MAX_WORLD + d;
    if (atomicAdd(ticket, 1u) == expected - 1) {
        *ticket = 0;  // everyone has arrived: re-arm for the next call
        if (d == p.rank) {
            st_release_gpu(seen_ptr(p, kFlagDispatch, p.rank), flag_value(p, 0));
        } else {
            fence_acq_rel_sys();
            st_relaxed_sys(flag_ptr(p.peer[d], p.off_flags, kFlagDispatch, p.rank), flag_value(p, 0));
        }
    }
}

// ---------------------------------------------------------------------------
// Watchers: warp i (lane 0) of the calling set polls the flag of `kind` written by the
// i-th peer after this rank and republishes it for the GPU.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void watcher_role(const DevParams& p, int kind, int phase, int set_warp) {
    if ((threadIdx.x & 31) != 0 || set_warp < 0 || set_warp >= p.ws - 1) return;
    const int peer = (p.rank + 1 + set_warp) % p.ws;
    watch_and_republish(p, kind, peer, phase, flag_value(p, 0));
}

// ---------------------------------------------------------------------------
// Sender blocks.  Shared-memory layout: ring | mbarriers | descriptors | token lists | warp totals.
// ---------------------------------------------------------------------------
struct SenderSmem {
    uint8_t* ring;
    unsigned long long* bars;
    SendDesc* desc;
    unsigned short* list;  // [ws][per]: this block's share of every destination's token list
    int* wt;
    int per;
};

__device__ __forceinline__ SenderSmem carve_sender(const DevParams& p, uint8_t* smem, int ns) {
    SenderSmem m;
    m.per = pipe_list_per(p.T_max, ns);
    m.ring = smem;
    m.bars = reinterpret_cast<unsigned long long*>(smem + (size_t)kStages * kStageBytes);
    m.desc = reinterpret_cast<SendDesc*>(smem + (size_t)kStages * kStageBytes + 128);
    m.list = reinterpret_cast<unsigned short*>(m.desc + 2 * kStages);
    m.wt = reinterpret_cast<int*>(smem + pipe_sender_smem(p.T_max, p.ws, ns) - 8 * A2A_MAX_WORLD * 4);
    return m;
}

// All threads: this block's share (wire rows n with n % ns == sb) of every destination's token
// list by ballot / popc compaction, and the total number of wire rows per destination in cnt[].
__device__ __forceinline__ void build_send_lists(const DevParams& p, const SenderSmem& m, int sb, int ns, int* cnt) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int base[A2A_MAX_WORLD];
#pragma unroll
    for (int d = 0; d < A2A_MAX_WORLD; ++d) base[d] = 0;
    for (int r0 = 0; r0 < p.T; r0 += kThreads) {
        const int t = r0 + tid;
        const unsigned mask = t < p.T ? dest_mask(p, t) : 0u;
#pragma unroll
        for (int d = 0; d < A2A_MAX_WORLD; ++d) {
            const unsigned b = __ballot_sync(0xffffffffu, (mask >> d) & 1u);
            if (lane == 0) m.wt[warp * A2A_MAX_WORLD + d] = __popc(b);
        }
        __syncthreads();
#pragma unroll
        for (int d = 0; d < A2A_MAX_WORLD; ++d) {
            const unsigned b = __ballot_sync(0xffffffffu, (mask >> d) & 1u);
            int before = 0, total = 0;
            for (int w = 0; w < kThreads / 32; ++w) {
                const int c = m.wt[w * A2A_MAX_WORLD + d];
                if (w < warp) before += c;
                total += c;
            }
            if ((mask >> d) & 1u) {
                const int n = base[d] + before + __popc(b & ((1u << lane) - 1u));
                if (n % ns == sb) m.list[d * m.per + n / ns] = (unsigned short)t;
            }
            base[d] += total;
        }
        __syncthreads();
    }
    if (tid == 0) {
#pragma unroll
        for (int d = 0; d < A2A_MAX_WORLD; ++d) cnt[d] = base[d];
    }
}

// A sender thread's destinations whose last store has been issued but not yet waited for, oldest
// first.  Bulk groups complete in order, so destination d (last group g_d) is through once at most
// (groups committed since g_d) groups are pending.  Nothing is waited for at a destination boundary:
// a destination is booked when its last store is `kArrivalLag` stores or `kArrivalAgeNs` old --
// by then the peer has acknowledged it, or nearly -- or at the end.  With one row per destination
// (small batches, many sender blocks) all rows leave back to back, and no flag waits for stores to
// OTHER destinations to pile up behind it.
constexpr long long kArrivalAgeNs = 2500;  // about one loaded NVLink round trip

struct PendingDests {
    int d[A2A_MAX_WORLD];
    long long g[A2A_MAX_WORLD];
    long long t[A2A_MAX_WORLD];
    int head = 0, tail = 0;
    __device__ __forceinline__ bool empty() const { return head == tail; }
    __device__ __forceinline__ void push(int dest, long long group) {
        d[tail % A2A_MAX_WORLD] = dest;
        g[tail % A2A_MAX_WORLD] = group;
        t[tail % A2A_MAX_WORLD] = global_ns();
        ++tail;
    }
    // Book every destination that is at least `lag` groups or kArrivalAgeNs old (lag 0: all of them);
    // `now` = groups committed so far.
    template <typename Arrive>
    __device__ __forceinline__ void drain(long long now, int lag, Arrive arrive) {
        const long long now_ns = head != tail ? global_ns() : 0;
        while (head != tail) {
            const int h = head % A2A_MAX_WORLD;
            const long long since = now - 1 - g[h];
            if (since < lag && now_ns - t[h] < kArrivalAgeNs) break;
            bulk_wait_done((int)min(since, 5LL));
            arrive(d[h]);
            ++head;
        }
    }
};

// Sender block `sb` of `ns`, 16-bit payload: all threads build the block's token lists; then
// thread 0 drives the copy engine (rows go HBM -> shared-memory ring -> peer without touching a
// register) while, if `watch_kind` >= 0, warps 1.. watch the peers' flags of that kind (they
// start only after the set-up barrier: a watcher may wait for a long time).
__device__ __forceinline__ void sender_role(const DevParams& p, uint8_t* smem, int sb, int ns, int watch_kind,
                                            int watch_phase) {
    const int tid = threadIdx.x, warp = tid >> 5;
    const SenderSmem m = carve_sender(p, smem, ns);
    uint8_t* ring = m.ring;
    unsigned long long* bars = m.bars;
    SendDesc* desc = m.desc;
    unsigned short* list = m.list;
    const int per = m.per;
    __shared__ int s_cnt[A2A_MAX_WORLD];
    if (tid == 0) {  // before the lists: thread 0 can issue its first loads the moment they are built
        for (int s = 0; s < kStages; ++s) mbar_init(smem_addr(bars + s), 1);
        mbar_fence_init();
    }
    build_send_lists(p, m, sb, ns, s_cnt);
    __syncthreads();
    stamp(p, kStampSetup + 0);
    if (tid != 0) {
        if (watch_kind >= 0 && warp > 0) watcher_role(p, watch_kind, watch_phase, warp - 1);
        return;
    }

    // ---- one thread drives the copy engine ----------------------------------------------
    const uint32_t expected = (uint32_t)(ns + p.routers);  // every sender block + the destination's router blocks
    auto arrive = [&](int d) {
        arrive_dest(p, d, expected);
        stamp(p, kStampDestDone + (d - p.rank + p.ws) % p.ws);
    };
    const int row_bytes = p.H * 2;
    const int pieces = (row_bytes + kStageBytes - 1) / kStageBytes;
    long long total = 0;
    for (int i = 1; i < p.ws; ++i) {
        const int d = (p.rank + i) % p.ws;
        const int mine = s_cnt[d] > sb ? (s_cnt[d] - sb + ns - 1) / ns : 0;
        if (mine == 0) arrive(d);  // nothing of ours goes there
        total += (long long)mine * pieces;
    }
    // A bulk store to a peer holds its stage until the peer has acknowledged the write (measured: with two
    // store stages a block moves 28 KB per ~1.5 us round trip whatever the link could take), local loads
    // complete in about a microsecond: two loads ahead, four stores in flight.
    constexpr int kLook = 2;
    int g_step = 1, g_i = 0, g_piece = 0;  // generator of the next piece to load
    auto skip_empty = [&] {
        while (g_step < p.ws) {
            const int d = (p.rank + g_step) % p.ws;
            const int mine = s_cnt[d] > sb ? (s_cnt[d] - sb + ns - 1) / ns : 0;
            if (g_i < mine) break;
            ++g_step;
            g_i = 0;
        }
    };
    skip_empty();
    PendingDests pending;
    bool failed = false;
    for (long long q = 0; q < total + kLook && !failed; ++q) {
        if (q < total) {
            const int st = (int)(q % kStages);
            if (q >= kStages) bulk_wait_read<kStages - kLook - 1>();  // the store that used this stage has read it
            const int d = (p.rank + g_step) % p.ws;
            const int mine = (s_cnt[d] - sb + ns - 1) / ns;
            const int n = sb + g_i * ns;  // wire row index at the destination
            const int t = list[d * per + g_i];
            const int off = g_piece * kStageBytes;
            const unsigned bytes = (unsigned)min(kStageBytes, row_bytes - off);
            const uint8_t* src = reinterpret_cast<const uint8_t*>(p.x) + (size_t)t * row_bytes + off;
            uint8_t* dst = p.peer[d] + p.off_stage + ((size_t)p.rank * p.T_max + n) * p.stage_row_bytes + off;
            const bool last_piece = (g_piece == pieces - 1);
            desc[st].dst = reinterpret_cast<unsigned long long>(dst);
            desc[st].bytes = bytes;
            desc[st].dest_done = (last_piece && g_i == mine - 1) ? d : -1;
            mbar_expect_tx(smem_addr(bars + st), bytes);
            bulk_load(smem_addr(ring + (size_t)st * kStageBytes), src, bytes, smem_addr(bars + st));
            if (q == 0) stamp(p, kStampSetup + 1);
            if (last_piece) {
                g_piece = 0;
                ++g_i;
                skip_empty();
            } else {
                ++g_piece;
            }
        }
        if (q >= kLook) {
            const long long it = q - kLook;
            const int st = (int)(it % kStages);
            const uint32_t parity = (uint32_t)((it / kStages) & 1);
            // the load is local and cannot be late by more than microseconds; bounded all the same
            long long t0 = 0;
            for (int spins = 0; !mbar_try_wait(smem_addr(bars + st), parity); ++spins) {
                if (spins == 0) t0 = global_ns();
                else if (global_ns() - t0 > p.timeout_ns) {
                    record_timeout(p, kPhaseSend, -1, p.epoch);
                    failed = true;
                    break;
                }
            }
            if (failed) break;
            bulk_store(reinterpret_cast<void*>(desc[st].dst), smem_addr(ring + (size_t)st * kStageBytes), desc[st].bytes);
            bulk_commit();
            if (it == 0) stamp(p, kStampSetup + 2);
            if (desc[st].dest_done >= 0) pending.push(desc[st].dest_done, it);  // group `it` was the destination's last
            pending.drain(it + 1, kArrivalLag, arrive);
        }
    }
    bulk_wait_done(0);  // nothing of ours is in flight when the block moves on
    if (!failed)
        while (!pending.empty()) pending.drain(1LL << 40, 0, arrive);
}

// Sender block `sb` of `ns`, FP8 payload: the whole block quantises one wire row at a time (the
// arithmetic -- an IEEE division per value -- is the cost here, so all eight warps share a row):
// 16-byte loads, amax over the 16 lanes of a 128-value block, e4m3 bytes and fp32 scales into one of
// eight 12 KB stages of the ring, then thread 0 hands the finished wire row to the copy engine and
// the block goes on to the next row while up to seven stores are still on their way.
constexpr int kFp8Stages = 8;
constexpr int kWarpStageBytes = kStages * kStageBytes / kFp8Stages;  // 12 KB: the largest FP8 wire row

template <typename T>
__device__ __forceinline__ void sender_role_fp8(const DevParams& p, uint8_t* smem, int sb, int ns) {
    const int tid = threadIdx.x;
    const SenderSmem m = carve_sender(p, smem, ns);
    __shared__ int s_cnt[A2A_MAX_WORLD];
    build_send_lists(p, m, sb, ns, s_cnt);
    __syncthreads();
    stamp(p, kStampSetup + 0);
    const uint32_t expected = (uint32_t)(ns + p.routers);
    auto arrive = [&](int d) {  // thread 0 only
        arrive_dest(p, d, expected);
        stamp(p, kStampDestDone + (d - p.rank + p.ws) % p.ws);
    };
    const int nvec = p.H >> 3;
    PendingDests pending;  // thread 0's bookkeeping, as in the 16-bit sender
    long long q = 0;       // rows this block has sent so far
    for (int i = 1; i < p.ws; ++i) {
        const int d = (p.rank + i) % p.ws;
        const int mine = s_cnt[d] > sb ? (s_cnt[d] - sb + ns - 1) / ns : 0;
        if (mine == 0) {
            if (tid == 0) arrive(d);  // nothing of ours goes there
            continue;
        }
        for (int g = 0; g < mine; ++g, ++q) {
            const int n = sb + g * ns;
            const int t = m.list[d * m.per + g];
            uint8_t* stage = m.ring + (size_t)(q % kFp8Stages) * kWarpStageBytes;
            if (tid == 0 && q >= kFp8Stages) bulk_wait_read<kFp8Stages - 1>();  // the store that used this stage has read it
            __syncthreads();
            const uint4* src = reinterpret_cast<const uint4*>(p.x) + (size_t)t * nvec;
            for (int v0 = 0; v0 < nvec; v0 += 4 * kThreads) {
                uint4 qv[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int v = v0 + u * kThreads + tid;
                    if (v < nvec) qv[u] = ld_input(src + v);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int v = v0 + u * kThreads + tid;  // nvec % 16 == 0: the 16 lanes of a scale block are all in or all out
                    float f[8];
                    float amax = 0.f;
                    if (v < nvec) {
                        unpack8<T>(qv[u], f);
#pragma unroll
                        for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(f[e]));
                    }
#pragma unroll
                    for (int o = 8; o >= 1; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
                    if (v < nvec) {
                        const float sc = amax > 0.f ? amax / 448.f : 1.f;
#pragma unroll
                        for (int e = 0; e < 8; ++e) f[e] = f[e] / sc;
                        reinterpret_cast<uint2*>(stage)[v] = pack8_e4m3(f);
                        if ((v & 15) == 0) reinterpret_cast<float*>(stage + p.H)[v >> 4] = sc;
                    }
                }
            }
            fence_async_smem();  // every thread's ordinary stores to the stage, before the copy engine reads it
            __syncthreads();
            if (tid == 0) {
                uint8_t* dst = p.peer[d] + p.off_stage + ((size_t)p.rank * p.T_max + n) * p.stage_row_bytes;
                bulk_store(dst, smem_addr(stage), (uint32_t)p.stage_row_bytes);
                bulk_commit();
                if (q == 0) stamp(p, kStampSetup + 2);
                if (g == mine - 1) pending.push(d, q);  // the block's last row for d
                pending.drain(q + 1, kArrivalLag, arrive);
            }
        }
    }
    if (tid == 0) {
        bulk_wait_done(0);
        while (!pending.empty()) pending.drain(1LL << 40, 0, arrive);
    }
}

// ---------------------------------------------------------------------------
// Router block `part` of `nparts` of destination rank d (all kThreads threads).  Every part
// builds the whole bitmap of d's experts (cheap, shared memory) but writes the records of its
// own slice of the tokens only (32-token words w with w % nparts == part): the scattered stores
// of one destination's records are spread over several SMs.  `first` marks the one router
// that books the pairs nobody owns (expert index out of range).
// ---------------------------------------------------------------------------
__device__ __forceinline__ void router_role(const DevParams& p, uint8_t* smem, int d, int part, int nparts, bool first,
                                            uint32_t expected) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int L = p.L, K = p.K, T = p.T;
    const int Wc = (T + 31) >> 5;
    unsigned* bits = reinterpret_cast<unsigned*>(smem);
    int* wpre = reinterpret_cast<int*>(smem) + (size_t)Wc * L;
    int* cnt = wpre + (size_t)Wc * L;
    int* wt = cnt + L;
    const int e0 = d * L;
    for (int i = tid; i < Wc * L; i += kThreads) bits[i] = 0u;
    __syncthreads();
    stamp(p, kStampStep + 0);
    for (int t = tid; t < T; t += kThreads) {
        const int* row = p.idx + (size_t)t * K;
        const unsigned bit = 1u << (t & 31);
        for (int k0 = 0; k0 < K; k0 += 8) {
            int e8[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) e8[u] = (k0 + u < K) ? __ldg(row + k0 + u) : e0;  // loaded together
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int k = k0 + u, e = e8[u];
                if (k >= K) break;
                if (e < 0 || e >= p.E) {
                    if (first) {
                        record_error(p.status, A2A_ERR_ROUTING, p.rank, -1, kPhaseRoute, p.epoch, e);
                        p.slot[(size_t)t * K + k] = -1;
                    }
                } else if (e >= e0 && e < e0 + L) {
                    if (atomicOr(bits + (size_t)(t >> 5) * L + (e - e0), bit) & bit)  // a repeat inside the token
                        if (part == 0) record_error(p.status, A2A_ERR_ROUTING, p.rank, -1, kPhaseRoute, p.epoch, e);
                }
            }
        }
    }
    __syncthreads();
    stamp(p, kStampStep + 1);
    for (int l = tid; l < L; l += kThreads) {
        int run = 0;
        for (int w = 0; w < Wc; ++w) {
            wpre[(size_t)w * L + l] = run;
            run += __popc(bits[(size_t)w * L + l]);
        }
        cnt[l] = run;
    }
    __syncthreads();
    stamp(p, kStampStep + 2);
    uint8_t* there = p.peer[d];
    int* rec_tok = reinterpret_cast<int*>(there + p.off_rec_tok) + (size_t)p.rank * p.T_max;
    unsigned* rec_ent = reinterpret_cast<unsigned*>(there + p.off_rec_ent) + (size_t)p.rank * p.T_max * K;
    float* rec_w = reinterpret_cast<float*>(there + p.off_rec_w) + (size_t)p.rank * p.T_max * K;
    int* meta = reinterpret_cast<int*>(there + p.off_meta);
    // Records, 256 tokens at a time.  First a thread per token: which tokens have a row at d, and by
    // ballot / popc compaction which wire row n each of them is.  Then a thread per (token, k) pair:
    // consecutive threads handle consecutive pairs, so the index / weight loads and the record stores
    // are coalesced and all warps of the block are busy even when its slice of the tokens is small.
    int* n_of = wt + 16; // [kThreads] wire row of the round's token, or -1 (not ours / no row at d)
    int base = 0;
    for (int r0 = 0; r0 < T; r0 += kThreads) {
        const int t = r0 + tid;
        bool has = false;
        if (t < T) {
            const int* row = p.idx + (size_t)t * K;
            for (int k = 0; k < K; ++k) {
                const int e = __ldg(row + k);
                has |= (e >= e0 && e < e0 + L);
            }
        }
        const unsigned b = __ballot_sync(0xffffffffu, has);
        if (lane == 0) wt[warp] = __popc(b);
        __syncthreads();
        int before = 0, total = 0;
        for (int w = 0; w < kThreads / 32; ++w) {
            if (w < warp) before += wt[w];
            total += wt[w];
        }
        int n = -1;
        if (has && ((t >> 5) % nparts) == part) {
            n = base + before + __popc(b & ((1u << lane) - 1u));  // wire row of token t at d
            rec_tok[n] = t;
        }
        n_of[tid] = n;
        base += total;
        __syncthreads();
        const int round_tokens = min(kThreads, T - r0);
        for (int q = tid; q < round_tokens * K; q += kThreads) {
            const int tl = q / K, k = q - tl * K;
            const int nn = n_of[tl];
            if (nn < 0) continue;
            const int tt = r0 + tl;
            const int* row = p.idx + (size_t)tt * K;
            const int e = __ldg(row + k);
            const float wk = __ldg(p.w + (size_t)tt * K + k);
            unsigned ent = kNoEntry;
            if (e >= e0 && e < e0 + L) {
                bool repeat = false;
                for (int kk = 0; kk < k; ++kk) repeat |= (__ldg(row + kk) == e);
                int j = -1;
                if (!repeat) {
                    const int l = e - e0, w = tt >> 5;
                    j = wpre[(size_t)w * L + l] + __popc(bits[(size_t)w * L + l] & ((1u << (tt & 31)) - 1u));
                    ent = ((unsigned)l << 16) | (unsigned)j;
                    meta[((size_t)l * p.ws + p.rank) * p.T_max + j] = (tt << 8) | k;
                }
                p.slot[(size_t)tt * K + k] = j;
            }
            rec_ent[(size_t)nn * K + k] = ent;
            rec_w[(size_t)nn * K + k] = wk;
        }
        __syncthreads();
    }
    if (part == 0) {
        int* counts = reinterpret_cast<int*>(there + p.off_counts) + (size_t)p.rank * kMaxChunks * L;
        for (int l = tid; l < L; l += kThreads) {
            counts[l] = cnt[l];
            p.send_counts[e0 + l] = cnt[l];
        }
        if (tid == 0) reinterpret_cast<int*>(there + p.off_hdr)[p.rank * 8] = base;
    }
    __syncthreads();
    stamp(p, kStampStep + 3);
    if (tid == 0) arrive_dest(p, d, expected);
}

// One 128-vector (2 KB) chunk of a wire row as four 16-byte vectors of T per lane.
// Own rows are read from x (FP8: through the same quantise / dequantise arithmetic the wire applies).
template <typename T, int PAYLOAD>
__device__ __forceinline__ void load_wire_chunk(const DevParams& p, bool own, const uint8_t* src, int v0, int nvec, uint4 (&q)[4]) {
    const int lane = threadIdx.x & 31;
    if (PAYLOAD != A2A_PAYLOAD_FP8) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int v = v0 + u * 32 + lane;
            if (v < nvec) q[u] = own ? ld_input(reinterpret_cast<const uint4*>(src) + v) : ld_stream(reinterpret_cast<const uint4*>(src) + v);
        }
    } else {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int v = v0 + u * 32 + lane;
            float f[8];
            if (own) {  // nvec % 16 == 0: the 16 lanes of a scale block are all in or all out
                float amax = 0.f;
                if (v < nvec) {
                    unpack8<T>(ld_input(reinterpret_cast<const uint4*>(src) + v), f);
#pragma unroll
                    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
                }
#pragma unroll
                for (int o = 8; o >= 1; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
                if (v < nvec) {
                    const float sc = amax > 0.f ? amax / 448.f : 1.f;
#pragma unroll
                    for (int i = 0; i < 8; ++i) f[i] = f[i] / sc;
                    unpack8_e4m3(pack8_e4m3(f), f);
#pragma unroll
                    for (int i = 0; i < 8; ++i) f[i] *= sc;
                    q[u] = pack8<T>(f);
                }
            } else if (v < nvec) {
                unpack8_e4m3(ld_stream(reinterpret_cast<const uint2*>(src) + v), f);
                const float sc = ld_stream(reinterpret_cast<const float*>(src + p.H) + (v >> 4));
#pragma unroll
                for (int i = 0; i < 8; ++i) f[i] *= sc;
                q[u] = pack8<T>(f);
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Expert block `xb` of `nxb`.  Sources are taken in arrival order (own rank first, then
// rank-1, rank-2, ...).  Inside a block the warps have fixed jobs so that no source ever waits
// for the bookkeeping of another:
//   warp 0  pollers: lane i waits for the dispatch flag of source position i, reads that source's
//           row count and raises a shared-memory word the workers spin on -- all sources at once,
//           so a batch whose rows are all there costs one flag latency, not one per source;
//   warp 1  completers: lane i waits until every worker warp has booked source i in a shared-memory
//           counter, fences (gpu scope; this is where the stores to the home rank are waited for) and
//           draws the block's ticket for that source -- the last ticket publishes the expert flag;
//   warps 2..7  workers: every worker warp of every expert block takes (wire row, 2 KB chunk) items
//           round-robin, continuing across sources where the previous one left off; having stored
//           its share of source i a warp fences at block scope, books the source and goes on to
//           source i+1 without waiting for anything.  PUSH: the partial row of a REMOTE token goes
//           home through the copy engine -- packed into one of the warp's two 2 KB shared-memory
//           slots and bulk-stored -- so that the back-pressure of the link never sits in the load /
//           store path of the SM in front of the slab stores and the next item's loads; such a source
//           is booked one source later (by then its bulk stores have long completed), the last at once.
// ---------------------------------------------------------------------------
constexpr int kExpertWorkers = kThreads / 32 - 2;

constexpr int kReturnSlotBytes = 2048;  // one 2 KB chunk of a partial row, two slots per worker warp

template <typename T, int PAYLOAD, bool PUSH>
__device__ __forceinline__ void expert_role(const DevParams& p, uint8_t* smem, int xb, int nxb) {
    __shared__ volatile int s_seen[A2A_MAX_WORLD];  // 0 waiting, 1 rows of source position i are here, -1 gave up
    __shared__ volatile int s_rows[A2A_MAX_WORLD];  // wire rows of source position i
    __shared__ int s_done[A2A_MAX_WORLD];           // worker warps that are through with source position i
    __shared__ volatile int s_dead;                 // a wait gave up: nothing further is published
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = p.K, nvec = p.H >> 3;
    const int nchunk = (nvec + 127) >> 7;
    const uint32_t want = flag_value(p, 0);
    uint8_t* self = p.peer[p.rank];
    if (tid < A2A_MAX_WORLD) {
        s_seen[tid] = 0;
        s_done[tid] = 0;
    }
    if (tid == 0) s_dead = 0;
    __syncthreads();
    if (warp == 0) {
        if (lane < p.ws) {
            const int i = lane, s = (p.rank - i + p.ws) % p.ws;
            const bool ok = wait_flag_gpu(seen_ptr(p, kFlagDispatch, s), want, p, kPhaseRecv, s);
            int n_s = 0;
            if (ok) {
                n_s = ld_stream(reinterpret_cast<const int*>(self + p.off_hdr) + s * 8);
                if (n_s < 0 || n_s > p.T_max) {
                    record_error(p.status, A2A_ERR_CAPACITY, p.rank, s, kPhaseExpert, p.epoch, n_s);
                    n_s = 0;
                }
            }
            s_rows[i] = n_s;
            __threadfence_block();
            s_seen[i] = ok ? 1 : -1;
            stamp_by(p, kStampSourceSeen + i, ok);
        }
        return;
    }
    if (warp == 1) {
        if (lane < p.ws) {
            const int i = lane, s = (p.rank - i + p.ws) % p.ws;
            while (*reinterpret_cast<volatile int*>(&s_done[i]) < kExpertWorkers) __nanosleep(40);  // bounded by the pollers' bounded waits
            if (!s_dead) {
                __threadfence();  // cumulative: the workers' stores, ordered before their bookings at block scope
                uint32_t* ticket = p.ptickets + kPipeTicketSource * A2A_MAX_WORLD + s;
                if (atomicAdd(ticket, 1u) == (uint32_t)nxb - 1u) {
                    *ticket = 0;
                    if (s == p.rank) {
                        st_release_gpu(seen_ptr(p, kFlagExpert, p.rank), want);
                    } else {
                        fence_acq_rel_sys();
                        st_relaxed_sys(flag_ptr(p.peer[s], p.off_flags, kFlagExpert, p.rank), want);
                    }
                }
                stamp_by(p, kStampSourceDone + i, true);
            }
        }
        return;
    }
    const int xw = xb * kExpertWorkers + (warp - 2);
    const int nxw = nxb * kExpertWorkers;
    const float scale = (float)(1 + p.rank);
    uint4* rows = reinterpret_cast<uint4*>(self + p.off_rows);
    uint8_t* slots = smem + (size_t)(warp - 2) * 2 * kReturnSlotBytes;  // this warp's two return slots
    auto book = [&](int i) {  // lane 0: this warp is through with source position i
        __threadfence_block();
        atomicAdd(&s_done[i], 1);
    };
    long long cursor = 0;
    int pending = -1;         // lane 0: a source whose bulk stores are still to be waited for
    long long groups = 0;     // lane 0: bulk groups this warp has committed so far
    long long pending_groups = 0;
    for (int i = 0; i < p.ws; ++i) {
        int seen;
        while ((seen = s_seen[i]) == 0) __nanosleep(40);  // bounded by the poller's own bounded wait
        if (seen < 0) {
            // nothing further is processed or published; the completers are still owed this warp's bookings
            if (lane == 0) {
                s_dead = 1;
                __threadfence_block();
                bulk_wait_done(0);
                if (pending >= 0) atomicAdd(&s_done[pending], 1);
                for (int j = i; j < p.ws; ++j) atomicAdd(&s_done[j], 1);
            }
            return;
        }
        const int s = (p.rank - i + p.ws) % p.ws;
        const int n_s = s_rows[i];
        const int* rec_tok = reinterpret_cast<const int*>(self + p.off_rec_tok) + (size_t)s * p.T_max;
        const unsigned* rec_ent = reinterpret_cast<const unsigned*>(self + p.off_rec_ent) + (size_t)s * p.T_max * K;
        const float* rec_w = reinterpret_cast<const float*>(self + p.off_rec_w) + (size_t)s * p.T_max * K;
        const bool own = (s == p.rank);
        const bool via_engine = PUSH && !own;  // the home rank is a peer: return through the copy engine
        const long long items = (long long)n_s * nchunk;
        for (long long it = (xw - cursor % nxw + nxw) % nxw; it < items; it += nxw) {
            const int n = (int)(it / nchunk), v0 = (int)(it - (long long)n * nchunk) * 128;
            const int t = ld_stream(rec_tok + n);
            const unsigned my_ent = lane < K ? (unsigned)ld_stream(reinterpret_cast<const int*>(rec_ent) + (size_t)n * K + lane) : kNoEntry;
            const float my_w = (PUSH && lane < K) ? ld_stream(rec_w + (size_t)n * K + lane) : 0.f;
            if (t < 0 || t >= p.T_max) {
                record_error(p.status, A2A_ERR_CAPACITY, p.rank, s, kPhaseRecv, p.epoch, t);
                continue;
            }
            const uint8_t* src = own ? reinterpret_cast<const uint8_t*>(p.x) + (size_t)t * p.H * 2
                                     : self + p.off_stage + ((size_t)s * p.T_max + n) * p.stage_row_bytes;
            uint4 q[4];
            load_wire_chunk<T, PAYLOAD>(p, own, src, v0, nvec, q);
            float acc[4][8];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                q[u] = scale8<T>(q[u], scale);  // the placeholder expert op: T(float(row) * (1 + rank))
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[u][e] = 0.f;
            }
            for (int k = 0; k < K; ++k) {
                const unsigned ent = __shfl_sync(0xffffffffu, my_ent, k);
                const float w = __shfl_sync(0xffffffffu, my_w, k);
                if (ent == kNoEntry) continue;
                const int l = (int)(ent >> 16), j = (int)(ent & 0xffffu);
                if (l >= p.L || j >= p.T_max) {
                    record_error(p.status, A2A_ERR_CAPACITY, p.rank, s, kPhaseExpert, p.epoch, (int)ent);
                    continue;
                }
                uint4* row = rows + (((size_t)l * p.ws + s) * p.T_max + j) * nvec;
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int v = v0 + u * 32 + lane;
                    if (v < nvec) {
                        st_stream(row + v, q[u]);
                        if (PUSH) {
                            float f[8];
                            unpack8<T>(q[u], f);
#pragma unroll
                            for (int e = 0; e < 8; ++e) acc[u][e] = fmaf(f[e], w, acc[u][e]);
                        }
                    }
                }
            }
            if (PUSH && !via_engine) {
                // one rank: the partial row IS the token's output -- no return buffer, no combine pass;
                // own tokens of several ranks: the return buffer is local memory
                uint4* home = p.ws == 1 ? reinterpret_cast<uint4*>(p.y) + (size_t)t * nvec
                                        : reinterpret_cast<uint4*>(self + p.off_ret) + ((size_t)p.rank * p.T_max + t) * nvec;
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int v = v0 + u * 32 + lane;
                    if (v < nvec) st_stream(home + v, pack8<T>(acc[u]));
                }
            }
            if (via_engine) {
                uint8_t* slot = slots + (size_t)(groups & 1) * kReturnSlotBytes;  // `groups` is warp-uniform: every lane counts
                if (groups >= 2) {
                    if (lane == 0) bulk_wait_read<1>();  // the store that used this slot two items ago has read it
                    __syncwarp();
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int v = v0 + u * 32 + lane;
                    if (v < nvec) reinterpret_cast<uint4*>(slot)[u * 32 + lane] = pack8<T>(acc[u]);
                }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) {
                    uint8_t* home = p.peer[s] + p.off_ret + (((size_t)p.rank * p.T_max + t) * nvec + v0) * 16;
                    bulk_store(home, smem_addr(slot), (uint32_t)(min(128, nvec - v0) * 16));
                    bulk_commit();
                }
                ++groups;
            }
        }
        cursor += items;
        __syncwarp();  // every lane's stores of this source precede lane 0's fence and booking
        if (lane == 0) {
            if (pending >= 0) {  // the source before: its bulk stores are at least this source's items old
                bulk_wait_done((int)min(groups - pending_groups, 5LL));
                fence_async_global();
                book(pending);
                pending = -1;
            }
            if (via_engine && i + 1 < p.ws) {
                pending = i;
                pending_groups = groups;
            } else {
                if (via_engine) {  // the last source: nothing comes after it to hide the wait behind
                    bulk_wait_done(0);
                    fence_async_global();
                }
                book(i);
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Combine at home, PUSH: y[t] = T(sum over the ranks d holding experts of t, ascending,
// of float(partial[d][t])).  Block `cb` of `ncb`; a warp per (token, 2 KB chunk).
// ---------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void combine_home_role(const DevParams& p, int cb, int ncb) {
    __shared__ int s_ok;
    const int tid = threadIdx.x, lane = tid & 31;
    const int K = p.K, nvec = p.H >> 3;
    const int nchunk = (nvec + 127) >> 7;
    const uint32_t want = flag_value(p, 0);
    if (p.ws == 1) {
        // The expert blocks have written y themselves.  What is left are tokens none of whose pairs is
        // valid (they have no wire row): their output is zero.  No flag is needed for that.
        const long long items = (long long)p.T * nchunk;
        const int cw = cb * (kThreads / 32) + (tid >> 5), ncw = ncb * (kThreads / 32);
        for (long long it = cw; it < items; it += ncw) {
            const int t = (int)(it / nchunk), v0 = (int)(it - (long long)t * nchunk) * 128;
            bool any = false;
            if (lane < K) {
                const int e = __ldg(p.idx + (size_t)t * K + lane);
                any = (e >= 0 && e < p.E);
            }
            if (__any_sync(0xffffffffu, any)) continue;
            uint4* y = reinterpret_cast<uint4*>(p.y) + (size_t)t * nvec;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int v = v0 + u * 32 + lane;
                if (v < nvec) st_stream(y + v, make_uint4(0u, 0u, 0u, 0u));
            }
        }
        stamp(p, kStampExpertSeen);
        stamp(p, kStampCombineDone);
        return;
    }
    if (tid < 32) {  // lane d waits for rank d's flag: all of them at once, not one after the other
        const bool ok = tid >= p.ws || wait_flag_gpu(seen_ptr(p, kFlagExpert, tid), want, p, kPhaseCombine, tid);
        const bool all = __all_sync(0xffffffffu, ok);
        if (tid == 0) s_ok = all ? 1 : 0;
    }
    __syncthreads();
    if (!s_ok) return;  // timeout recorded; y is left untouched
    stamp(p, kStampExpertSeen);
    const uint4* ret = reinterpret_cast<const uint4*>(p.peer[p.rank] + p.off_ret);
    // a warp per (token, 2 KB chunk): four vectors per lane of up to four contributing ranks' partial rows
    // are requested before the first is used (sixteen loads in flight), ranks 0-3 then 4-7, added in rank order
    const long long items = (long long)p.T * nchunk;
    const int cw = cb * (kThreads / 32) + (tid >> 5), ncw = ncb * (kThreads / 32);
    for (long long it = cw; it < items; it += ncw) {
        const int t = (int)(it / nchunk), v0 = (int)(it - (long long)t * nchunk) * 128;
        unsigned bit = 0u;
        if (lane < K) {
            const int e = __ldg(p.idx + (size_t)t * K + lane);
            if (e >= 0 && e < p.E) bit = 1u << (e / p.L);
        }
        const unsigned mask = __reduce_or_sync(0xffffffffu, bit);
        float acc[4][8];
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[u][e] = 0.f;
#pragma unroll
        for (int g = 0; g < A2A_MAX_WORLD; g += 4) {
            if (((mask >> g) & 0xfu) == 0u) continue;
            uint4 q[4][4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if ((mask >> (g + j)) & 1u) {
                    const uint4* row = ret + ((size_t)(g + j) * p.T_max + t) * nvec;
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int v = v0 + u * 32 + lane;
                        if (v < nvec) q[j][u] = ld_stream(row + v);
                    }
                }
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if ((mask >> (g + j)) & 1u) {
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int v = v0 + u * 32 + lane;
                        if (v < nvec) {
                            float f[8];
                            unpack8<T>(q[j][u], f);
#pragma unroll
                            for (int e = 0; e < 8; ++e) acc[u][e] += f[e];
                        }
                    }
                }
        }
        uint4* y = reinterpret_cast<uint4*>(p.y) + (size_t)t * nvec;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int v = v0 + u * 32 + lane;
            if (v < nvec) st_stream(y + v, pack8<T>(acc[u]));
        }
    }
    __syncthreads();
    stamp(p, kStampCombineDone);
}

// PULL combine never reads a rank it has no pair on, but a rank may only start its next call
// once EVERY peer is through with this one's records; one thread sees to that.
__device__ __forceinline__ void wait_all_experts(const DevParams& p) {
    if (blockIdx.x == 0 && threadIdx.x == 0)
        for (int d = 0; d < p.ws; ++d)
            if (!wait_flag_gpu(seen_ptr(p, kFlagExpert, d), flag_value(p, 0), p, kPhaseCombine, d)) break;
}

// ---------------------------------------------------------------------------
// Kernels
// ---------------------------------------------------------------------------
extern __shared__ __align__(128) uint8_t a2a_pipe_smem[];

// Block mapping.  16-bit payloads: blocks [0, senders) send, 0 and 1 also carry the watchers in
// their spare warps.  FP8: every warp of a sender block quantises, so blocks 0 and 1 only watch
// and blocks [2, 2 + senders) send.  The next `ws` blocks route first, and every block after
// the senders is an expert block.
template <int PAYLOAD>
__device__ __forceinline__ int watcher_blocks(const DevParams& p) { return (PAYLOAD == A2A_PAYLOAD_FP8 && p.ws > 1) ? 2 : 0; }

// The whole path in one cooperative launch.
template <typename T, int PAYLOAD, bool PUSH>
__global__ void __launch_bounds__(kThreads, 2) pipe_forward_kernel(const __grid_constant__ DevParams p) {
    const int G = (int)gridDim.x, b = (int)blockIdx.x;
    const int ns = p.ws > 1 ? p.senders : 0;
    const int nw = watcher_blocks<PAYLOAD>(p);
    stamp(p, kStampStart);
    if (b < nw) {
        stamp_value(p, kStampRole, kRoleWatcher);
        watcher_role(p, b == 0 ? kFlagDispatch : kFlagExpert, b == 0 ? kPhaseRecv : kPhaseCombine, (int)(threadIdx.x >> 5));
    } else if (b < nw + ns) {
        if (PAYLOAD == A2A_PAYLOAD_FP8) {
            stamp_value(p, kStampRole, kRoleSender);
            sender_role_fp8<T>(p, a2a_pipe_smem, b - nw, ns);
        } else {
            stamp_value(p, kStampRole, b < 2 ? (kRoleSender | kRoleWatcher) : kRoleSender);
            sender_role(p, a2a_pipe_smem, b, ns, b == 0 ? kFlagDispatch : (b == 1 ? kFlagExpert : -1),
                        b == 0 ? kPhaseRecv : kPhaseCombine);
        }
        stamp(p, kStampSent);
    } else {
        const int xb = b - nw - ns, nxb = G - nw - ns;
        if (xb < p.ws * p.routers) {  // router part xb / ws of destination rank+1+(xb % ws): first needed, first served
            const int d = (p.rank + 1 + xb % p.ws) % p.ws;
            router_role(p, a2a_pipe_smem, d, xb / p.ws, p.routers, xb == 0, (uint32_t)(d == p.rank ? 0 : ns) + p.routers);
            stamp(p, kStampSent);
        }
        stamp_value(p, kStampRole, xb < p.ws * p.routers ? (kRoleExpert | kRoleRouter) : kRoleExpert);
        expert_role<T, PAYLOAD, PUSH>(p, a2a_pipe_smem, xb, nxb);
    }
    __syncthreads();
    stamp(p, kStampExpertDone);
    if (PUSH) {
        combine_home_role<T>(p, b, G);
    } else {
        combine_phase<T>(p, b, G, /*own_watchers=*/false);
        wait_all_experts(p);
    }
}

// The same roles as separate launches, for stepping several ranks on ONE GPU (a kernel that
// waits never shares the GPU with the kernel it waits for) and for callers that want the
// phases apart.  ROLE 0: senders + routers.  1: one watcher block + experts.  2: one
// watcher block + combine.
template <typename T, int PAYLOAD, bool PUSH, int ROLE>
__global__ void __launch_bounds__(kThreads, 2) pipe_role_kernel(const __grid_constant__ DevParams p) {
    const int G = (int)gridDim.x, b = (int)blockIdx.x;
    const int ns = p.ws > 1 ? p.senders : 0;
    stamp(p, kStampStart);
    if (ROLE == 0) {
        if (b < ns) {
            if (PAYLOAD == A2A_PAYLOAD_FP8) sender_role_fp8<T>(p, a2a_pipe_smem, b, ns);
            else sender_role(p, a2a_pipe_smem, b, ns, -1, 0);
        } else {
            const int rb = b - ns, d = (p.rank + 1 + rb % p.ws) % p.ws;
            router_role(p, a2a_pipe_smem, d, rb / p.ws, p.routers, rb == 0, (uint32_t)(d == p.rank ? 0 : ns) + p.routers);
        }
        stamp(p, kStampSent);
    } else if (ROLE == 1) {
        if (b == 0) watcher_role(p, kFlagDispatch, kPhaseRecv, (int)(threadIdx.x >> 5));
        else expert_role<T, PAYLOAD, PUSH>(p, a2a_pipe_smem, b - 1, G - 1);
        stamp(p, kStampExpertDone);
    } else {
        if (b == 0) {
            watcher_role(p, kFlagExpert, kPhaseCombine, (int)(threadIdx.x >> 5));
        } else if (PUSH) {
            combine_home_role<T>(p, b - 1, G - 1);
        } else {
            combine_phase<T>(p, b - 1, G - 1, /*own_watchers=*/false);
        }
        if (!PUSH) wait_all_experts(p);
    }
}

}  // namespace a2a
