// The hot-path kernels: routing, dispatch (send / receive), expert placeholder,
// combine, plus the export and barrier helpers.  Hand-written for sm_100a; all of
// them are bound by NVLink or HBM bandwidth (there is no contraction on this path),
// so they are built from 16-byte vector accesses, grids sized in multiples of the
// 148 SMs, and flag traffic kept off the critical path.
#pragma once

#include "a2a_device.cuh"

namespace a2a {

constexpr int kRouteThreads = 1024;
constexpr int kRowThreads = 256;      // threads that move one row together
constexpr int kCombineThreads = 128;  // threads per (token, chunk) item
constexpr int kCombineChunk = kCombineThreads * 8;  // elements per combine item

enum Ticket : int { kTicketSend = 0, kTicketExpert = 1 };

// ---------------------------------------------------------------------------
// K1 routing.  One block walks the (token, k) pairs in order, 1024 per step:
// a warp match gives each pair its rank among the equal experts of its warp,
// a per-expert exclusive scan over the 32 warp counts (plus the running total
// of earlier steps) gives the warp's base.  slot[p] = number of earlier pairs
// of this rank with the same expert -- the position the CPU reference gives the
// row inside one source's contribution (reference.py:79-86, :140-146).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kRouteThreads) route_kernel(const __grid_constant__ DevParams p) {
    extern __shared__ int smem[];
    int* warp_cnt = smem;             // [32][E]
    int* running = smem + 32 * p.E;   // [E]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int E = p.E, P = p.T * p.K;
    for (int e = tid; e < E; e += kRouteThreads) running[e] = 0;
    for (int p0 = 0; p0 < P; p0 += kRouteThreads) {
        for (int i = tid; i < 32 * E; i += kRouteThreads) warp_cnt[i] = 0;
        __syncthreads();
        const int pair = p0 + tid;
        int e = -1;
        if (pair < P) {
            e = p.idx[pair];
            if (e < 0 || e >= E) {
                record_error(p.status, A2A_ERR_ROUTING, p.rank, -1, kPhaseRoute, p.epoch, e);
                e = -1;
            }
        }
        const unsigned same = __match_any_sync(0xffffffffu, e);
        const int before = __popc(same & ((1u << lane) - 1u));
        if (e >= 0 && before == 0) warp_cnt[warp * E + e] = __popc(same);
        __syncthreads();
        for (int ee = tid; ee < E; ee += kRouteThreads) {
            int run = running[ee];
#pragma unroll 8
            for (int w = 0; w < 32; ++w) {
                const int c = warp_cnt[w * E + ee];
                warp_cnt[w * E + ee] = run;
                run += c;
            }
            running[ee] = run;
        }
        __syncthreads();
        if (pair < P) {
            int s = -1;
            if (e >= 0) {
                s = warp_cnt[warp * E + e] + before;
                if (s >= p.T_max) {
                    record_error(p.status, A2A_ERR_CAPACITY, p.rank, -1, kPhaseRoute, p.epoch, e);
                    s = -1;
                }
            }
            p.slot[pair] = s;
        }
        __syncthreads();
    }
    for (int e = tid; e < E; e += kRouteThreads) p.send_counts[e] = min(running[e], p.T_max);
}

// Publish this rank's per-expert counts and the dispatch flag to every peer.
// Called by all threads of the one block that arrived last.
__device__ __forceinline__ void publish_dispatch(const DevParams& p) {
    const int tid = threadIdx.x;
    for (int e = tid; e < p.E; e += blockDim.x) {
        const int d = e / p.L, l = e - d * p.L;
        int* counts = reinterpret_cast<int*>(p.peer[d] + p.off_counts);
        counts[p.rank * p.L + l] = p.send_counts[e];
    }
    __threadfence_system();
    __syncthreads();
    if (tid < p.ws) st_release_sys(flag_ptr(p.peer[tid], p.off_flags, kFlagDispatch, p.rank), p.epoch);
}

// ---------------------------------------------------------------------------
// K2 dispatch, sending half, DIRECT payload.  One block per (token, k) pair at a
// time: 256 threads read the row from HBM/L2 with up to four 16-byte loads each in
// flight and store it straight into slab (expert, this rank) of the expert's rank
// (NVLink for a peer, HBM for ourselves).  The last block to finish publishes.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kRowThreads) dispatch_send_direct_kernel(const __grid_constant__ DevParams p) {
    const int tid = threadIdx.x;
    const int P = p.T * p.K;
    const int nvec = p.H >> 3;
    for (int pair = blockIdx.x; pair < P; pair += gridDim.x) {
        const int j = p.slot[pair];
        if (j < 0) continue;
        const int e = p.idx[pair];
        const int d = e / p.L, l = e - d * p.L;
        const int t = pair / p.K, k = pair - t * p.K;
        const size_t row = ((size_t)l * p.ws + p.rank) * p.T_max + j;
        const uint4* src = reinterpret_cast<const uint4*>(p.x) + (size_t)t * nvec;
        uint4* dst = reinterpret_cast<uint4*>(p.peer[d] + p.off_rows) + row * nvec;
        for (int v0 = 0; v0 < nvec; v0 += kRowThreads * 4) {
            uint4 r[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int v = v0 + u * kRowThreads + tid;
                if (v < nvec) r[u] = ld_input(src + v);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int v = v0 + u * kRowThreads + tid;
                if (v < nvec) st_stream(dst + v, r[u]);
            }
        }
        if (tid == 0) reinterpret_cast<int*>(p.peer[d] + p.off_meta)[row] = (t << 8) | k;
    }
    if (grid_arrive_last(p.tickets + kTicketSend)) publish_dispatch(p);
}

// ---------------------------------------------------------------------------
// K3 dispatch receiving half / expert placeholder.  Template switches:
//   WAIT    wait for every source's dispatch flag of this call (bounded)
//   SCALE   run the placeholder expert op in place on the valid rows
//   PUBLISH tell every home rank that this rank's expert outputs are ready
// The valid rows of all (local expert, source) slabs are flattened with a prefix
// sum over the received counts so that skewed routing does not idle blocks.
// ---------------------------------------------------------------------------
template <typename T, bool WAIT, bool SCALE, bool PUBLISH>
__global__ void __launch_bounds__(kRowThreads) expert_rows_kernel(const __grid_constant__ DevParams p) {
    __shared__ int prefix[A2A_MAX_EXPERTS + 1];
    __shared__ int s_ok;
    const int tid = threadIdx.x;
    uint8_t* self = p.peer[p.rank];
    if (tid == 0) s_ok = 1;
    __syncthreads();
    if (WAIT) {
        if (tid < p.ws) {
            if (!wait_flag(flag_ptr(self, p.off_flags, kFlagDispatch, tid), p.epoch, p, kPhaseRecv, tid)) s_ok = 0;
        }
        __syncthreads();
    }
    if (!s_ok) return;  // error recorded; nothing is published, peers run into their own budget
    const int nslab = p.L * p.ws;  // slab i = l * ws + s
    if (WAIT || SCALE) {
        const int* counts = reinterpret_cast<const int*>(self + p.off_counts);
        for (int i = tid; i < nslab; i += kRowThreads) {
            const int l = i / p.ws, s = i - l * p.ws;
            int c = __ldcg(counts + s * p.L + l);
            if (c < 0 || c > p.T_max) {
                record_error(p.status, A2A_ERR_CAPACITY, p.rank, s, kPhaseRecv, p.epoch, c);
                c = 0;
            }
            prefix[i] = c;
        }
        block_exclusive_scan(prefix, nslab);
        if (blockIdx.x == 0)
            for (int l = tid; l < p.L; l += kRowThreads) p.expert_count[l] = prefix[(l + 1) * p.ws] - prefix[l * p.ws];
    }
    if (SCALE) {
        const int total = prefix[nslab];
        const int nvec = p.H >> 3;
        const float scale = (float)(1 + p.rank);
        uint4* rows = reinterpret_cast<uint4*>(self + p.off_rows);
        for (int r = blockIdx.x; r < total; r += gridDim.x) {
            const int i = upper_slab(prefix, nslab, r);
            const int j = r - prefix[i];
            uint4* row = rows + ((size_t)i * p.T_max + j) * nvec;
            for (int v0 = 0; v0 < nvec; v0 += kRowThreads * 4) {
                uint4 q[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int v = v0 + u * kRowThreads + tid;
                    if (v < nvec) q[u] = ld_stream(row + v);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int v = v0 + u * kRowThreads + tid;
                    if (v < nvec) {
                        float f[8];
                        unpack8<T>(q[u], f);
#pragma unroll
                        for (int c = 0; c < 8; ++c) f[c] *= scale;
                        st_stream(row + v, pack8<T>(f));
                    }
                }
            }
        }
    }
    if (PUBLISH) {
        if (grid_arrive_last(p.tickets + kTicketExpert)) {
            if (tid < p.ws) st_release_sys(flag_ptr(p.peer[tid], p.off_flags, kFlagExpert, p.rank), p.epoch);
        }
    }
}

// ---------------------------------------------------------------------------
// K4 combine (pull).  Item = (token, 1024-element chunk); 128 threads, each owns 8
// consecutive elements: it loads the 16 bytes of each of the token's K expert
// outputs from the rank that holds them (the slot is known from routing, so there
// is no metadata to fetch), accumulates float(row) * w[t,k] in fp32 registers in k
// order and stores 16 bytes of y.  Loads are issued four at a time.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kCombineThreads) combine_kernel(const __grid_constant__ DevParams p) {
    __shared__ const uint4* s_row[A2A_MAX_TOPK];
    __shared__ float s_w[A2A_MAX_TOPK];
    __shared__ int s_ok;
    const int tid = threadIdx.x;
    if (tid == 0) s_ok = 1;
    __syncthreads();
    if (tid < p.ws) {
        if (!wait_flag(flag_ptr(p.peer[p.rank], p.off_flags, kFlagExpert, tid), p.epoch, p, kPhaseCombine, tid)) s_ok = 0;
    }
    __syncthreads();
    if (!s_ok) return;
    const int nvec = p.H >> 3;
    const int nchunk = (p.H + kCombineChunk - 1) / kCombineChunk;
    const int items = p.T * nchunk;
    const int K = p.K;
    for (int item = blockIdx.x; item < items; item += gridDim.x) {
        const int t = item / nchunk, c = item - t * nchunk;
        __syncthreads();
        if (tid < K) {
            const int pair = t * K + tid;
            const int j = p.slot[pair];
            const uint4* row = nullptr;
            float w = 0.f;
            if (j >= 0) {
                const int e = p.idx[pair];
                const int d = e / p.L, l = e - d * p.L;
                row = reinterpret_cast<const uint4*>(p.peer[d] + p.off_rows) +
                      (((size_t)l * p.ws + p.rank) * p.T_max + j) * nvec;
                w = p.w[pair];
            }
            s_row[tid] = row;
            s_w[tid] = w;
        }
        __syncthreads();
        const int v = c * kCombineThreads + tid;
        if (v < nvec) {
            float acc[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = 0.f;
            for (int k0 = 0; k0 < K; k0 += 4) {
                uint4 q[4];
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (k0 + u < K && s_row[k0 + u] != nullptr) q[u] = ld_stream(s_row[k0 + u] + v);
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (k0 + u < K && s_row[k0 + u] != nullptr) {
                        float f[8];
                        unpack8<T>(q[u], f);
                        const float w = s_w[k0 + u];
#pragma unroll
                        for (int i = 0; i < 8; ++i) acc[i] = fmaf(f[i], w, acc[i]);
                    }
            }
            st_stream(reinterpret_cast<uint4*>(p.y) + (size_t)t * nvec + v, pack8<T>(acc));
        }
    }
}

// ---------------------------------------------------------------------------
// Export: the reference's dispatch return value (reference.py:148) packed from the
// slabs -- rows of one expert ordered by (source rank, token, k).  Test helper.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kRowThreads) export_dispatch_kernel(const __grid_constant__ DevParams p, int* out_counts, uint4* out_rows,
                                                                     int* out_meta) {
    __shared__ int prefix[A2A_MAX_EXPERTS + 1];
    const int tid = threadIdx.x;
    uint8_t* self = p.peer[p.rank];
    const int nslab = p.L * p.ws;
    const int* counts = reinterpret_cast<const int*>(self + p.off_counts);
    for (int i = tid; i < nslab; i += kRowThreads) {
        const int l = i / p.ws, s = i - l * p.ws;
        int c = counts[s * p.L + l];
        prefix[i] = (c < 0 || c > p.T_max) ? 0 : c;
    }
    block_exclusive_scan(prefix, nslab);
    if (blockIdx.x == 0)
        for (int l = tid; l < p.L; l += kRowThreads) out_counts[l] = prefix[(l + 1) * p.ws] - prefix[l * p.ws];
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
        for (int v = tid; v < nvec; v += kRowThreads) out_rows[out_row * nvec + v] = rows[in_row * nvec + v];
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
        wait_flag(flag_ptr(p.peer[p.rank], p.off_flags, kFlagBarrier, tid), barrier_epoch, p, kPhaseBarrier, tid);
    }
}

}  // namespace a2a
