// liba2a.so -- host side of the C ABI declared in include/a2a.h: context life cycle,
// symmetric-region layout, CUDA-IPC peer mapping and kernel launches.  No torch
// types, no allocation and no host synchronisation on the data path.
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <new>

#include "a2a.h"
#include "a2a_kernels.cuh"
#include "a2a_pipe.cuh"

using namespace a2a;

namespace {

constexpr int kTraceBlocks = 2048;  // blocks the in-kernel trace buffer has room for
constexpr size_t kMaxSmemBytes = 200 * 1024;  // routing bitmap budget per block (227 KB is the sm_100 limit)
constexpr size_t kMaxPipeSmemBytes = 100 * 1024;  // pipelined kernels: two blocks per SM must fit

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct Layout {
    size_t off_rows, off_meta, off_counts, off_flags, off_stage, total;
    size_t off_rec_tok, off_rec_ent, off_rec_w, off_hdr, off_ret;  // pipelined schedule only
    int stage_row_bytes;
};

// What every rank of a group must agree on, appended to the IPC handle each rank exports.
struct Fingerprint {
    uint32_t magic;
    int32_t world_size, num_experts, experts_per_token, hidden_dim, max_num_tokens, dtype, payload, schedule, combine,
        chunks;
    uint32_t pad;
    uint64_t layout_total;
};
constexpr uint32_t kFingerprintMagic = 0x41324131u;  // "A2A1"
constexpr size_t kHandleBlobBytes = 128;             // CUDA IPC handle (64) + fingerprint, padded
static_assert(sizeof(cudaIpcMemHandle_t) + sizeof(Fingerprint) <= kHandleBlobBytes, "handle blob too small");

Layout make_layout(const a2a_config& c) {
    Layout l{};
    const size_t L = c.num_experts / c.world_size, ws = c.world_size, T = c.max_num_tokens, H = c.hidden_dim;
    size_t off = 0;
    l.off_rows = off;
    off = align_up(off + L * ws * T * H * 2, 256);
    l.off_meta = off;  // everything from here up to the wire rows starts as zero
    off = align_up(off + L * ws * T * sizeof(int32_t), 256);
    l.off_counts = off;
    off = align_up(off + ws * kMaxChunks * L * sizeof(int32_t), 256);
    l.off_flags = off;
    off = align_up(off + (size_t)kNumFlagKinds * A2A_MAX_WORLD * kFlagStride * sizeof(uint32_t), 256);
    l.stage_row_bytes = 0;
    l.off_stage = off;
    if (c.payload != A2A_PAYLOAD_DIRECT) {
        l.stage_row_bytes = (int)(c.payload == A2A_PAYLOAD_FP8 ? align_up(H + 4 * (H / kFp8Block), 16) : H * 2);
        off = align_up(off + ws * T * (size_t)l.stage_row_bytes, 256);
    }
    l.off_rec_tok = l.off_rec_ent = l.off_rec_w = l.off_hdr = l.off_ret = off;
    if (c.schedule == A2A_SCHEDULE_PIPELINED) {
        const size_t K = c.experts_per_token;
        l.off_rec_tok = off;  off = align_up(off + ws * T * 4, 256);
        l.off_rec_ent = off;  off = align_up(off + ws * T * K * 4, 256);
        l.off_rec_w = off;    off = align_up(off + ws * T * K * 4, 256);
        l.off_hdr = off;      off = align_up(off + ws * 8 * 4, 256);
        l.off_ret = off;
        if (c.combine == A2A_COMBINE_PUSH) off = align_up(off + ws * T * H * 2, 256);
    }
    l.total = off;
    return l;
}

}  // namespace

struct a2a_ctx {
    a2a_config cfg;
    Layout lay;
    DevParams p;            // template of the kernel parameter block (per-call fields patched at launch)
    uint8_t* region;        // our symmetric region (cudaMalloc)
    uint8_t* scratch;       // local scratch (cudaMalloc)
    size_t scratch_bytes;
    void* ipc_mapped[A2A_MAX_WORLD];  // peers opened through CUDA IPC (to close on destroy)
    bool peers_ready;
    bool routed, sent;
    uint32_t epoch, barrier_epoch;
    int cur_tokens;
    int64_t launches;
    cudaStream_t side;      // private stream for status reads
    int* host_code;         // mapped host word mirroring the device status code
    // device staging for the host-buffer entry point
    void* h_x;
    int32_t* h_idx;
    float* h_w;
    void* h_y;
    int smem_bytes;         // dynamic shared memory of the routing-carrying kernels
    int num_sms;
    int forward_grid;       // co-resident grid of the one-launch kernel
    int pipe_smem;          // dynamic shared memory of the pipelined kernels
    bool fused;             // a2a_forward uses the one-launch kernel
    bool plain_launch;      // A2A_LAUNCH=plain: ordinary instead of cooperative launch of the one-launch kernels
    char errmsg[160];       // detail of the last host-detected error
    long long* trace;       // device trace buffer (always allocated, used only while tracing is on)
    int last_grid;          // grid of the most recent traced launch
};

namespace {

#define CUDA_TRY(expr)                                   \
    do {                                                 \
        cudaError_t e_ = (expr);                         \
        if (e_ != cudaSuccess) return -(int)e_;          \
    } while (0)

struct DeviceGuard {
    int prev = -1;
    bool changed = false;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) == cudaSuccess && prev != dev) {
            changed = (cudaSetDevice(dev) == cudaSuccess);
        }
    }
    ~DeviceGuard() {
        if (changed) cudaSetDevice(prev);
    }
};

// Token chunks a context really uses: whole 32-token words, at most as many as there are words.
int resolved_chunks(const a2a_config& c) {
    const int Wmax = (c.max_num_tokens + 31) / 32;
    const int chunks = c.chunks >= 1 ? c.chunks : 1;
    return chunks < Wmax ? chunks : Wmax;
}

Fingerprint fingerprint_of(const a2a_config& c) {
    Fingerprint f;
    memset(&f, 0, sizeof(f));
    f.magic = kFingerprintMagic;
    f.world_size = c.world_size; f.num_experts = c.num_experts; f.experts_per_token = c.experts_per_token;
    f.hidden_dim = c.hidden_dim; f.max_num_tokens = c.max_num_tokens; f.dtype = c.dtype;
    f.payload = c.payload; f.schedule = c.schedule; f.combine = c.combine; f.chunks = resolved_chunks(c);
    f.layout_total = make_layout(c).total;
    return f;
}

// The gathered blobs against this rank's configuration; fills msg on a mismatch.
int check_blobs(const a2a_config& cfg, const uint8_t* all, size_t nbytes, char* msg, size_t msg_len) {
    if (msg && msg_len) msg[0] = 0;
    if (nbytes != (size_t)cfg.world_size * kHandleBlobBytes) {
        if (msg) snprintf(msg, msg_len, "handle blobs: got %zu bytes, expected %zu (%d ranks x %zu)", nbytes,
                          (size_t)cfg.world_size * kHandleBlobBytes, cfg.world_size, kHandleBlobBytes);
        return A2A_ERR_CONFIG;
    }
    const Fingerprint mine = fingerprint_of(cfg);
    for (int r = 0; r < cfg.world_size; ++r) {
        Fingerprint f;
        memcpy(&f, all + (size_t)r * kHandleBlobBytes + sizeof(cudaIpcMemHandle_t), sizeof(f));
        if (memcmp(&f, &mine, sizeof(f)) != 0) {
            if (msg) snprintf(msg, msg_len, "rank %d was created with a different configuration than rank %d%s", r,
                              cfg.rank, f.magic != kFingerprintMagic ? " (or its handle blob is damaged)" : "");
            return A2A_ERR_CONFIG;
        }
    }
    return A2A_OK;
}

// Sender blocks of the pipelined kernel.  16-bit payload: one thread per block drives the copy
// engine (two 14 KB loads ahead, four stores in flight).  Measured at 8 GPUs, the sending role alone
// takes 52 us + 624 us / blocks (78 / 65 / 63 / 60 us with 24 / 48 / 64 / 96 blocks) and the whole
// call 126.7 / 113.8 / 110.6 / 109.1 us: 96 blocks at 8 ranks, where there is most to send; 48 below,
// where the call is a chain of latencies and the expert blocks are better served.  FP8: a block
// quantises a row at a time and the arithmetic is the cost: 96.
int pipe_senders(const a2a_config& c) {
    if (c.world_size == 1) return 0;
    if (c.senders > 0) return c.senders;
    return (c.payload == A2A_PAYLOAD_FP8 || c.world_size >= 8) ? 96 : 48;
}

int validate(const a2a_config& c) {
    if (c.world_size < 1 || c.world_size > A2A_MAX_WORLD) return A2A_ERR_CONFIG;
    if (c.rank < 0 || c.rank >= c.world_size) return A2A_ERR_CONFIG;
    if (c.num_experts < 1 || c.num_experts > A2A_MAX_EXPERTS || c.num_experts % c.world_size != 0) return A2A_ERR_CONFIG;
    if (c.experts_per_token < 1 || c.experts_per_token > A2A_MAX_TOPK || c.experts_per_token > c.num_experts)
        return A2A_ERR_CONFIG;
    if (c.hidden_dim < 8 || c.hidden_dim % 8 != 0) return A2A_ERR_CONFIG;
    if (c.max_num_tokens < 1) return A2A_ERR_CONFIG;
    if (c.dtype != A2A_DTYPE_BF16 && c.dtype != A2A_DTYPE_FP16) return A2A_ERR_CONFIG;
    if (c.payload != A2A_PAYLOAD_DIRECT && c.payload != A2A_PAYLOAD_DEDUP && c.payload != A2A_PAYLOAD_FP8)
        return A2A_ERR_CONFIG;
    if (c.max_num_tokens > 65535) return A2A_ERR_CONFIG;  // slots travel in 16 bits
    if (c.payload == A2A_PAYLOAD_FP8 && c.hidden_dim % kFp8Block != 0) return A2A_ERR_CONFIG;
    if (block_smem_ints(c.num_experts, c.max_num_tokens, c.experts_per_token) * sizeof(int) > kMaxSmemBytes) return A2A_ERR_CONFIG;
    if (c.device < 0) return A2A_ERR_CONFIG;
    if (c.schedule != A2A_SCHEDULE_PHASED && c.schedule != A2A_SCHEDULE_PIPELINED) return A2A_ERR_CONFIG;
    if (c.combine != A2A_COMBINE_PULL && c.combine != A2A_COMBINE_PUSH) return A2A_ERR_CONFIG;
    if (c.chunks < 0 || c.chunks > kMaxChunks || c.senders < 0 || c.senders > 128) return A2A_ERR_CONFIG;
    if (c.combine == A2A_COMBINE_PUSH && c.schedule != A2A_SCHEDULE_PIPELINED) return A2A_ERR_CONFIG;
    if (c.schedule == A2A_SCHEDULE_PIPELINED) {
        // the senders move one wire row per (token, destination): the per-pair DIRECT payload has none
        if (c.payload != A2A_PAYLOAD_DEDUP && c.payload != A2A_PAYLOAD_FP8) return A2A_ERR_CONFIG;
        // FP8: a warp assembles a whole wire row in its own stage of the sender ring
        if (c.payload == A2A_PAYLOAD_FP8 && make_layout(c).stage_row_bytes > kWarpStageBytes) return A2A_ERR_CONFIG;
        if (c.chunks > 1) return A2A_ERR_CONFIG;
        const int senders = pipe_senders(c);
        if (c.world_size > 1 && senders < 2) return A2A_ERR_CONFIG;  // blocks 0 and 1 carry the watchers
        if (pipe_sender_smem(c.max_num_tokens, c.world_size, senders) > kMaxPipeSmemBytes ||
            pipe_router_smem(c.max_num_tokens, c.num_experts / c.world_size) > kMaxPipeSmemBytes)
            return A2A_ERR_CONFIG;
    }
    return A2A_OK;
}

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

// Rows are moved as 16-byte vectors and by the copy engine: both need 16-byte alignment.
inline bool rows_aligned(const void* ptr) { return reinterpret_cast<uintptr_t>(ptr) % 16 == 0; }

inline int grid_for(const a2a_ctx* c, long long items, int per_sm) {
    long long cap = (long long)c->num_sms * per_sm;
    long long g = items < cap ? items : cap;
    return g < 1 ? 1 : (int)g;
}

DevParams call_params(a2a_ctx* c) {
    DevParams p = c->p;
    p.T = c->cur_tokens;
    p.epoch = c->epoch;
    return p;
}

// ---- kernel selection by (element type, payload) ---------------------------
template <template <typename, int> class F, typename... A>
auto select_tp(const a2a_ctx* c, A... a) {
    const bool bf = c->cfg.dtype == A2A_DTYPE_BF16;
    switch (c->cfg.payload) {
        case A2A_PAYLOAD_DEDUP:
            return bf ? F<__nv_bfloat16, A2A_PAYLOAD_DEDUP>::get(a...) : F<__half, A2A_PAYLOAD_DEDUP>::get(a...);
        case A2A_PAYLOAD_FP8:
            return bf ? F<__nv_bfloat16, A2A_PAYLOAD_FP8>::get(a...) : F<__half, A2A_PAYLOAD_FP8>::get(a...);
        default:
            return bf ? F<__nv_bfloat16, A2A_PAYLOAD_DIRECT>::get(a...) : F<__half, A2A_PAYLOAD_DIRECT>::get(a...);
    }
}

using KernelFn = void (*)(DevParams);
template <typename T, int P> struct SendSel { static KernelFn get() { return send_kernel<T, P>; } };
template <typename T, int P> struct ForwardSel { static KernelFn get() { return forward_kernel<T, P>; } };
template <typename T, int P> struct ExpertSel {
    // the receive-side launches of the public phases
    static KernelFn get(bool wait, bool fanout, bool scale, bool publish) {
        if (wait && fanout && scale && publish) return expert_kernel<T, P, true, true, true, true>;      // recv + expert fused
        if (wait && fanout && !scale && !publish) return expert_kernel<T, P, true, true, false, false>;  // dispatch_recv
        if (!wait && !fanout && scale && publish) return expert_kernel<T, P, false, false, true, true>;  // expert_placeholder
        return expert_kernel<T, P, false, false, false, true>;                                           // expert_done
    }
};
// pipelined schedule: (element type, payload, push/pull) -> kernel; role -1 = the one-launch kernel
template <typename T, int P, bool PUSH>
KernelFn pipe_fn_tp(int role) {
    switch (role) {
        case 0: return pipe_role_kernel<T, P, PUSH, 0>;
        case 1: return pipe_role_kernel<T, P, PUSH, 1>;
        case 2: return pipe_role_kernel<T, P, PUSH, 2>;
        default: return pipe_forward_kernel<T, P, PUSH>;
    }
}
template <typename T>
KernelFn pipe_fn_t(const a2a_ctx* c, int role) {
    const bool push = c->cfg.combine == A2A_COMBINE_PUSH;
    if (c->cfg.payload == A2A_PAYLOAD_FP8)
        return push ? pipe_fn_tp<T, A2A_PAYLOAD_FP8, true>(role) : pipe_fn_tp<T, A2A_PAYLOAD_FP8, false>(role);
    return push ? pipe_fn_tp<T, A2A_PAYLOAD_DEDUP, true>(role) : pipe_fn_tp<T, A2A_PAYLOAD_DEDUP, false>(role);
}
KernelFn pipe_fn(const a2a_ctx* c, int role) {
    return c->cfg.dtype == A2A_DTYPE_BF16 ? pipe_fn_t<__nv_bfloat16>(c, role) : pipe_fn_t<__half>(c, role);
}

KernelFn combine_fn(const a2a_ctx* c) {
    return c->cfg.dtype == A2A_DTYPE_BF16 ? (KernelFn)combine_kernel<__nv_bfloat16> : (KernelFn)combine_kernel<__half>;
}

int launch(a2a_ctx* c, KernelFn fn, int grid, int smem, cudaStream_t st, bool cooperative = false) {
    DevParams p = call_params(c);
    if (p.trace != nullptr && grid > kTraceBlocks) p.trace = nullptr;
    if (p.trace != nullptr) c->last_grid = grid;
    void* args[] = {&p};
    cudaError_t e = (cooperative && !c->plain_launch)
        ? cudaLaunchCooperativeKernel((const void*)fn, dim3(grid), dim3(kThreads), args, smem, st)
        : cudaLaunchKernel((const void*)fn, dim3(grid), dim3(kThreads), args, smem, st);
    c->launches++;
    if (e != cudaSuccess) return -(int)e;
    return A2A_OK;
}

int begin_call(a2a_ctx* c, const int32_t* idx, int T) {
    if (!c->peers_ready) return A2A_ERR_STATE;
    if (T < 0 || T > c->cfg.max_num_tokens || (T > 0 && idx == nullptr)) return A2A_ERR_CONFIG;
    if (reinterpret_cast<uintptr_t>(idx) % 4 != 0) return A2A_ERR_CONFIG;
    c->epoch++;
    c->cur_tokens = T;
    c->p.idx = idx;
    c->routed = true;
    c->sent = false;
    return A2A_OK;
}

int do_route(a2a_ctx* c, const int32_t* idx, int T, cudaStream_t st) {
    int r = begin_call(c, idx, T);
    if (r != A2A_OK) return r;
    return launch(c, route_kernel, 1, c->smem_bytes, st);
}

int do_send(a2a_ctx* c, const void* x, cudaStream_t st) {
    if (!c->routed || c->sent) return A2A_ERR_STATE;
    if (c->cur_tokens > 0 && x == nullptr) return A2A_ERR_CONFIG;
    if (!rows_aligned(x)) return A2A_ERR_CONFIG;
    c->p.x = x;
    const long long items = (long long)c->cur_tokens *
        (c->cfg.payload == A2A_PAYLOAD_DIRECT ? c->cfg.experts_per_token : c->cfg.world_size);
    int r = launch(c, select_tp<SendSel>(c), grid_for(c, items, 8), c->smem_bytes, st);
    if (r == A2A_OK) c->sent = true;
    return r;
}

// grid of the receive-side kernels: a multiple of the world size so every source gets the same share
int expert_grid(const a2a_ctx* c, int per_sm) {
    const int ws = c->cfg.world_size;
    int g = c->num_sms * per_sm;
    g = (g / ws) * ws;
    return g < ws ? ws : g;
}

int do_expert(a2a_ctx* c, bool wait, bool fanout, bool scale, bool publish, int grid, cudaStream_t st) {
    if (!c->sent) return A2A_ERR_STATE;
    return launch(c, select_tp<ExpertSel>(c, wait, fanout, scale, publish), grid, c->smem_bytes, st);
}

int do_combine(a2a_ctx* c, const float* w, void* y, cudaStream_t st) {
    if (!c->sent) return A2A_ERR_STATE;
    if (c->cur_tokens > 0 && (w == nullptr || y == nullptr)) return A2A_ERR_CONFIG;
    if (!rows_aligned(y) || reinterpret_cast<uintptr_t>(w) % 4 != 0) return A2A_ERR_CONFIG;
    c->p.w = w;
    c->p.y = y;
    const int nseg = (c->cfg.hidden_dim / 8 + 63) / 64;  // a warp per (token, 1 KB segment)
    const long long warps = (long long)c->cur_tokens * nseg;
    return launch(c, combine_fn(c), grid_for(c, (warps + kThreads / 32 - 1) / (kThreads / 32), 8), 0, st);
}

}  // namespace

extern "C" {

const char* a2a_strerror(int status) {
    switch (status) {
        case A2A_OK: return "ok";
        case A2A_ERR_CONFIG: return "invalid configuration or argument";
        case A2A_ERR_CAPACITY: return "slab capacity exceeded (an expert got more than max_num_tokens rows from one source)";
        case A2A_ERR_TIMEOUT: return "a device-side wait on a peer ran out of its time budget";
        case A2A_ERR_STATE: return "call order violated";
        case A2A_ERR_ROUTING: return "expert index out of range";
        default: break;
    }
    if (status < 0) return cudaGetErrorString((cudaError_t)(-status));
    return "unknown status";
}

size_t a2a_ipc_handle_bytes(void) { return kHandleBlobBytes; }

const char* a2a_last_error(a2a_ctx* c) { return c ? c->errmsg : "no context"; }

int a2a_fingerprint(const a2a_config* cfg, uint8_t* out) {
    if (cfg == nullptr || out == nullptr) return A2A_ERR_CONFIG;
    int v = validate(*cfg);
    if (v != A2A_OK) return v;
    memset(out, 0, kHandleBlobBytes - sizeof(cudaIpcMemHandle_t));
    const Fingerprint f = fingerprint_of(*cfg);
    memcpy(out, &f, sizeof(f));
    return A2A_OK;
}

int a2a_check_handles(const a2a_config* cfg, const uint8_t* all, size_t nbytes, char* msg, size_t msg_len) {
    if (cfg == nullptr || all == nullptr) return A2A_ERR_CONFIG;
    return check_blobs(*cfg, all, nbytes, msg, msg_len);
}

int a2a_create(a2a_ctx** out, const a2a_config* cfg) {
    if (out == nullptr || cfg == nullptr) return A2A_ERR_CONFIG;
    *out = nullptr;
    int v = validate(*cfg);
    if (v != A2A_OK) return v;
    int ndev = 0;
    CUDA_TRY(cudaGetDeviceCount(&ndev));
    if (cfg->device >= ndev) return A2A_ERR_CONFIG;
    DeviceGuard guard(cfg->device);

    a2a_ctx* c = new (std::nothrow) a2a_ctx();
    if (c == nullptr) return -(int)cudaErrorMemoryAllocation;
    memset(c, 0, sizeof(*c));
    c->cfg = *cfg;
    if (c->cfg.timeout_ms <= 0) c->cfg.timeout_ms = 2000;
    c->lay = make_layout(c->cfg);
    const int E = cfg->num_experts, K = cfg->experts_per_token, T = cfg->max_num_tokens, H = cfg->hidden_dim;
    const int L = E / cfg->world_size;

    cudaError_t e = cudaMalloc(&c->region, c->lay.total);
    if (e != cudaSuccess) { delete c; return -(int)e; }
    // every flag word starts at zero = "epoch 0, nothing has happened" (the staged wire rows need no clearing)
    cudaMemset(c->region + c->lay.off_meta, 0, c->lay.off_stage - c->lay.off_meta);

    // local scratch: slot | send_counts | tickets | seen words | status | trace | host-path staging
    size_t off = 0;
    const size_t o_slot = off;      off = align_up(off + (size_t)T * K * 4, 256);
    const size_t o_send = off;      off = align_up(off + (size_t)E * 4, 256);
    const size_t o_tick = off;      off = align_up(off + 8 * 4, 256);
    const size_t o_ptick = off;     off = align_up(off + 2 * A2A_MAX_WORLD * 4, 256);
    const size_t o_seen = off;      off = align_up(off + 2 * A2A_MAX_WORLD * kFlagStride * 4, 256);
    const size_t o_stat = off;      off = align_up(off + sizeof(StatusBlock), 256);
    const size_t o_trace = off;     off = align_up(off + (size_t)kTraceBlocks * kNumStamps * 8, 256);
    const size_t o_hx = off;        off = align_up(off + (size_t)T * H * 2, 256);
    const size_t o_hy = off;        off = align_up(off + (size_t)T * H * 2, 256);
    const size_t o_hidx = off;      off = align_up(off + (size_t)T * K * 4, 256);
    const size_t o_hw = off;        off = align_up(off + (size_t)T * K * 4, 256);
    c->scratch_bytes = off;
    e = cudaMalloc(&c->scratch, off);
    if (e != cudaSuccess) { cudaFree(c->region); delete c; return -(int)e; }
    cudaMemset(c->scratch, 0, off);
    e = cudaStreamCreateWithFlags(&c->side, cudaStreamNonBlocking);
    if (e != cudaSuccess) { cudaFree(c->scratch); cudaFree(c->region); delete c; return -(int)e; }
    e = cudaHostAlloc(reinterpret_cast<void**>(&c->host_code), 64, cudaHostAllocMapped);
    if (e != cudaSuccess) { cudaStreamDestroy(c->side); cudaFree(c->scratch); cudaFree(c->region); delete c; return -(int)e; }
    *c->host_code = 0;
    {
        StatusBlock sb;
        memset(&sb, 0, sizeof(sb));
        sb.host_code = c->host_code;  // unified addressing: the host pointer is valid on the device
        cudaMemcpy(c->scratch + o_stat, &sb, sizeof(sb), cudaMemcpyHostToDevice);
    }

    DevParams& p = c->p;
    p.peer[cfg->rank] = c->region;
    p.off_rows = c->lay.off_rows; p.off_meta = c->lay.off_meta; p.off_counts = c->lay.off_counts;
    p.off_flags = c->lay.off_flags; p.off_stage = c->lay.off_stage;
    p.off_rec_tok = c->lay.off_rec_tok; p.off_rec_ent = c->lay.off_rec_ent; p.off_rec_w = c->lay.off_rec_w;
    p.off_hdr = c->lay.off_hdr; p.off_ret = c->lay.off_ret;
    p.stage_row_bytes = c->lay.stage_row_bytes;
    p.senders = pipe_senders(c->cfg);
    {
        // router blocks per destination: about 32 in all, never more than there are 32-token words
        const int words = (T + 31) / 32;
        int r = 32 / cfg->world_size;
        if (r > 8) r = 8;
        if (r > words) r = words;
        p.routers = r < 1 ? 1 : r;
    }
    p.rank = cfg->rank; p.ws = cfg->world_size; p.E = E; p.K = K; p.H = H; p.T_max = T; p.L = L;
    p.timeout_ns = (long long)c->cfg.timeout_ms * 1000000LL;
    {
        // Token chunks the call is pipelined in (whole 32-token words).  Default 1: measured on
        // B200 the per-chunk publication (a ticket round and a system fence each) costs more than
        // the overlap returns -- c4, DEDUP: 32.7 / 37.5 / 59.3 us with 1 / 2 / 4 chunks on one GPU,
        // 70.7 / 68.1 / 89.3 us on two.  cfg.chunks = 2..4 opts in; every rank of a group must agree
        // (the value is part of the fingerprint the ranks exchange).
        const int Wmax = (T + 31) / 32;
        const int chunks = resolved_chunks(*cfg);
        p.wpc = (Wmax + chunks - 1) / chunks;
        p.chunks = (Wmax + p.wpc - 1) / p.wpc;
    }
    p.slot = reinterpret_cast<int*>(c->scratch + o_slot);
    p.send_counts = reinterpret_cast<int*>(c->scratch + o_send);
    p.tickets = reinterpret_cast<uint32_t*>(c->scratch + o_tick);
    p.ptickets = reinterpret_cast<uint32_t*>(c->scratch + o_ptick);
    p.seen = reinterpret_cast<uint32_t*>(c->scratch + o_seen);
    p.status = reinterpret_cast<a2a_status_t*>(c->scratch + o_stat);
    c->trace = reinterpret_cast<long long*>(c->scratch + o_trace);
    c->h_x = c->scratch + o_hx; c->h_y = c->scratch + o_hy;
    c->h_idx = reinterpret_cast<int32_t*>(c->scratch + o_hidx);
    c->h_w = reinterpret_cast<float*>(c->scratch + o_hw);

    // Kernel attributes are per function and device, not per context: opt every routing-carrying
    // kernel in for the whole shared-memory budget, then size this context's own launches.
    c->smem_bytes = (int)(block_smem_ints(E, T, K) * sizeof(int));
    KernelFn fns[] = {route_kernel, select_tp<SendSel>(c), select_tp<ForwardSel>(c),
                      select_tp<ExpertSel>(c, true, true, true, true), select_tp<ExpertSel>(c, true, true, false, false),
                      select_tp<ExpertSel>(c, false, false, true, true), select_tp<ExpertSel>(c, false, false, false, true)};
    for (KernelFn fn : fns) {
        e = cudaFuncSetAttribute((const void*)fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxSmemBytes);
        if (e != cudaSuccess) break;
    }
    int coop = 0, occ = 0;
    const bool pipelined = cfg->schedule == A2A_SCHEDULE_PIPELINED;
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&c->num_sms, cudaDevAttrMultiProcessorCount, cfg->device);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, cfg->device);
    if (pipelined) {
        const size_t a = pipe_sender_smem(T, cfg->world_size, p.senders), b = pipe_router_smem(T, L);
        c->pipe_smem = (int)align_up(a > b ? a : b, 128);
        for (int role = -1; role <= 2 && e == cudaSuccess; ++role)
            e = cudaFuncSetAttribute((const void*)pipe_fn(c, role), cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)kMaxPipeSmemBytes);
        if (e == cudaSuccess)
            e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, (const void*)pipe_fn(c, -1), kThreads, c->pipe_smem);
        if (e == cudaSuccess) {
            if (occ > 2) occ = 2;
            c->forward_grid = c->num_sms * occ;
            c->fused = true;
            // the one launch needs every block resident and room for the roles: senders, one router per
            // destination, and at least as many expert blocks again
            const int watchers = (cfg->payload == A2A_PAYLOAD_FP8 && cfg->world_size > 1) ? 2 : 0;
            if (coop == 0 || c->forward_grid < watchers + p.senders + 2 * cfg->world_size * p.routers) {
                a2a_destroy(c);
                return A2A_ERR_CONFIG;
            }
        }
    } else if (e == cudaSuccess) {
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, (const void*)select_tp<ForwardSel>(c), kThreads,
                                                          c->smem_bytes);
        if (e == cudaSuccess) {
            if (occ > 8) occ = 8;
            c->forward_grid = c->num_sms * occ;
            c->fused = (coop != 0 && occ >= 1);
        }
    }
    if (e == cudaSuccess) e = cudaDeviceSynchronize();  // memsets done before any peer may write here
    if (e != cudaSuccess) { a2a_destroy(c); return -(int)e; }
    {
        // Opt-in, for measurement: launch the one-launch kernels like any other kernel.  The grid is sized
        // to be co-resident either way, but only the cooperative launch makes the driver GUARANTEE it; with
        // an ordinary launch a grid that did not get all its blocks running at once ends in
        // A2A_ERR_TIMEOUT (every wait is bounded), not in a hang.
        const char* env = getenv("A2A_LAUNCH");
        c->plain_launch = (env != nullptr && strcmp(env, "plain") == 0);
    }
    c->peers_ready = (cfg->world_size == 1);
    *out = c;
    return A2A_OK;
}

int a2a_destroy(a2a_ctx* c) {
    if (c == nullptr) return A2A_OK;
    DeviceGuard guard(c->cfg.device);
    cudaDeviceSynchronize();
    for (int r = 0; r < A2A_MAX_WORLD; ++r)
        if (c->ipc_mapped[r]) cudaIpcCloseMemHandle(c->ipc_mapped[r]);
    if (c->side) cudaStreamDestroy(c->side);
    if (c->host_code) cudaFreeHost(c->host_code);
    if (c->scratch) cudaFree(c->scratch);
    if (c->region) cudaFree(c->region);
    delete c;
    return A2A_OK;
}

int a2a_export_handle(a2a_ctx* c, uint8_t* out) {
    if (c == nullptr || out == nullptr) return A2A_ERR_CONFIG;
    DeviceGuard guard(c->cfg.device);
    cudaIpcMemHandle_t h;
    CUDA_TRY(cudaIpcGetMemHandle(&h, c->region));
    memset(out, 0, kHandleBlobBytes);
    memcpy(out, &h, sizeof(h));
    const Fingerprint f = fingerprint_of(c->cfg);
    memcpy(out + sizeof(h), &f, sizeof(f));
    return A2A_OK;
}

int a2a_open_peers(a2a_ctx* c, const uint8_t* all, size_t nbytes) {
    if (c == nullptr || all == nullptr) return A2A_ERR_CONFIG;
    if (c->peers_ready && c->cfg.world_size > 1) return A2A_ERR_STATE;
    // every rank must have been created with the same problem, payload and schedule: a rank that
    // differs would lay its region out differently and the peers would write into the wrong places
    const int chk = check_blobs(c->cfg, all, nbytes, c->errmsg, sizeof(c->errmsg));
    if (chk != A2A_OK) return chk;
    DeviceGuard guard(c->cfg.device);
    for (int r = 0; r < c->cfg.world_size; ++r) {
        if (r == c->cfg.rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, all + (size_t)r * kHandleBlobBytes, sizeof(h));
        void* ptr = nullptr;
        CUDA_TRY(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
        c->ipc_mapped[r] = ptr;
        c->p.peer[r] = static_cast<uint8_t*>(ptr);
    }
    c->peers_ready = true;
    return A2A_OK;
}

int a2a_attach_local_peers(a2a_ctx* c, a2a_ctx* const* peers) {
    if (c == nullptr || peers == nullptr) return A2A_ERR_CONFIG;
    DeviceGuard guard(c->cfg.device);
    for (int r = 0; r < c->cfg.world_size; ++r) {
        a2a_ctx* q = peers[r];
        if (q == nullptr || q->cfg.rank != r) return A2A_ERR_CONFIG;
        const Fingerprint a = fingerprint_of(c->cfg), b = fingerprint_of(q->cfg);
        if (memcmp(&a, &b, sizeof(a)) != 0) {
            snprintf(c->errmsg, sizeof(c->errmsg), "rank %d was created with a different configuration than rank %d", r,
                     c->cfg.rank);
            return A2A_ERR_CONFIG;
        }
        if (q->cfg.device != c->cfg.device) {
            cudaError_t e = cudaDeviceEnablePeerAccess(q->cfg.device, 0);
            if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
            else if (e != cudaSuccess) return -(int)e;
        }
        c->p.peer[r] = q->region;
    }
    c->peers_ready = true;
    return A2A_OK;
}

int a2a_route(a2a_ctx* c, const int32_t* idx, int T, void* stream) {
    if (c == nullptr) return A2A_ERR_CONFIG;
    DeviceGuard guard(c->cfg.device);
    return do_route(c, idx, T, as_stream(stream));
}

int a2a_dispatch_send(a2a_ctx* c, const void* x, void* stream) {
    if (c == nullptr) return A2A_ERR_CONFIG;
    DeviceGuard guard(c->cfg.device);
    return do_send(c, x, as_stream(stream));
}

int a2a_dispatch_recv(a2a_ctx* c, void* stream) {
    if (c == nullptr) return A2A_ERR_CONFIG;
    DeviceGuard guard(c->cfg.device);
    // DIRECT: the rows are already in place; a minimal grid just waits for every source
    const int grid = c->cfg.payload == A2A_PAYLOAD_DIRECT ? c->cfg.world_size : expert_grid(c, 4);
    return do_expert(c, true, true, false, false, grid, as_stream(stream));
}

int a2a_expert_placeholder(a2a_ctx* c, void* stream) {
    if (c == nullptr) return A2A_ERR_CONFIG;
    DeviceGuard guard(c->cfg.device);
    return do_expert(c, false, false, true, true, expert_grid(c, 4), as_stream(stream));
}

int a2a_dispatch_recv_expert(a2a_ctx* c, void* stream) {
    if (c == nullptr) return A2A_ERR_CONFIG;
    DeviceGuard guard(c->cfg.device);
    return do_expert(c, true, true, true, true, expert_grid(c, 4), as_stream(stream));
}

int a2a_expert_done(a2a_ctx* c, void* stream) {
    if (c == nullptr) return A2A_ERR_CONFIG;
    DeviceGuard guard(c->cfg.device);
    return do_expert(c, false, false, false, true, expert_grid(c, 1), as_stream(stream));
}

int a2a_combine(a2a_ctx* c, const float* w, void* y, void* stream) {
    if (c == nullptr) return A2A_ERR_CONFIG;
    DeviceGuard guard(c->cfg.device);
    return do_combine(c, w, y, as_stream(stream));
}

int a2a_set_fused(a2a_ctx* c, int on) {
    if (c == nullptr) return A2A_ERR_CONFIG;
    if (on && c->forward_grid < 1) return A2A_ERR_STATE;
    c->fused = (on != 0);
    return A2A_OK;
}

int a2a_forward(a2a_ctx* c, const void* x, const int32_t* idx, const float* w, void* y, int T, void* stream) {
    if (c == nullptr) return A2A_ERR_CONFIG;
    DeviceGuard guard(c->cfg.device);
    cudaStream_t st = as_stream(stream);
    int r = begin_call(c, idx, T);
    if (r != A2A_OK) return r;
    if (T > 0 && (x == nullptr || w == nullptr || y == nullptr)) return A2A_ERR_CONFIG;
    if (!rows_aligned(x) || !rows_aligned(y) || reinterpret_cast<uintptr_t>(w) % 4 != 0) return A2A_ERR_CONFIG;
    if (c->cfg.schedule == A2A_SCHEDULE_PIPELINED) {
        c->p.x = x;
        c->p.w = w;
        c->p.y = y;
        r = launch(c, pipe_fn(c, -1), c->forward_grid, c->pipe_smem, st, /*cooperative=*/true);
        if (r == A2A_OK) c->sent = true;
        return r;
    }
    if (c->fused) {
        c->p.x = x;
        c->p.w = w;
        c->p.y = y;
        r = launch(c, select_tp<ForwardSel>(c), c->forward_grid, c->smem_bytes, st, /*cooperative=*/true);
        if (r == A2A_OK) c->sent = true;
        return r;
    }
    r = do_send(c, x, st);
    if (r != A2A_OK) return r;
    r = do_expert(c, true, true, true, true, expert_grid(c, 4), st);
    if (r != A2A_OK) return r;
    return do_combine(c, w, y, st);
}

int a2a_forward_host(a2a_ctx* c, const void* x, const int32_t* idx, const float* w, void* y, int T, void* stream) {
    if (c == nullptr) return A2A_ERR_CONFIG;
    if (T < 0 || T > c->cfg.max_num_tokens) return A2A_ERR_CONFIG;
    if (T > 0 && (x == nullptr || idx == nullptr || w == nullptr || y == nullptr)) return A2A_ERR_CONFIG;
    DeviceGuard guard(c->cfg.device);
    cudaStream_t st = as_stream(stream);
    const size_t row = (size_t)c->cfg.hidden_dim * 2, tk = (size_t)T * c->cfg.experts_per_token * 4;
    if (T > 0) {
        CUDA_TRY(cudaMemcpyAsync(c->h_idx, idx, tk, cudaMemcpyHostToDevice, st));
        CUDA_TRY(cudaMemcpyAsync(c->h_x, x, row * T, cudaMemcpyHostToDevice, st));
        CUDA_TRY(cudaMemcpyAsync(c->h_w, w, tk, cudaMemcpyHostToDevice, st));
    }
    int r = a2a_forward(c, c->h_x, c->h_idx, c->h_w, c->h_y, T, stream);
    if (r != A2A_OK) return r;
    if (T > 0) CUDA_TRY(cudaMemcpyAsync(y, c->h_y, row * T, cudaMemcpyDeviceToHost, st));
    return A2A_OK;
}

int a2a_pipe_step(a2a_ctx* c, int role, const void* x, const int32_t* idx, const float* w, void* y, int T, void* stream) {
    if (c == nullptr || role < 0 || role > 2) return A2A_ERR_CONFIG;
    if (c->cfg.schedule != A2A_SCHEDULE_PIPELINED) return A2A_ERR_STATE;
    DeviceGuard guard(c->cfg.device);
    cudaStream_t st = as_stream(stream);
    const int ws = c->cfg.world_size;
    if (role == 0) {
        int r = begin_call(c, idx, T);
        if (r != A2A_OK) return r;
        if (T > 0 && (x == nullptr || w == nullptr || y == nullptr)) return A2A_ERR_CONFIG;
        if (!rows_aligned(x) || !rows_aligned(y) || reinterpret_cast<uintptr_t>(w) % 4 != 0) return A2A_ERR_CONFIG;
        c->p.x = x;
        c->p.w = w;
        c->p.y = y;  // with one rank and the PUSH combine the expert blocks already write the output
        r = launch(c, pipe_fn(c, 0), c->p.senders + ws * c->p.routers, c->pipe_smem, st);
        if (r == A2A_OK) c->sent = true;
        return r;
    }
    if (!c->sent) return A2A_ERR_STATE;
    return launch(c, pipe_fn(c, role), 1 + c->num_sms * 2, c->pipe_smem, st);
}

int a2a_barrier(a2a_ctx* c, void* stream) {
    if (c == nullptr) return A2A_ERR_CONFIG;
    if (!c->peers_ready) return A2A_ERR_STATE;
    DeviceGuard guard(c->cfg.device);
    c->barrier_epoch++;
    barrier_kernel<<<1, 32, 0, as_stream(stream)>>>(call_params(c), c->barrier_epoch);
    c->launches++;
    CUDA_TRY(cudaGetLastError());
    return A2A_OK;
}

int a2a_link_probe(a2a_ctx* c, int peer, size_t bytes, void* stream) {
    if (c == nullptr || peer < 0 || peer >= c->cfg.world_size) return A2A_ERR_CONFIG;
    if (!c->peers_ready) return A2A_ERR_STATE;
    const size_t room = c->lay.off_meta - c->lay.off_rows;  // the slab rows: dead between calls
    if (bytes == 0 || bytes > room) return A2A_ERR_CONFIG;
    DeviceGuard guard(c->cfg.device);
    CUDA_TRY(cudaMemcpyAsync(c->p.peer[peer] + c->lay.off_rows, c->region + c->lay.off_rows, bytes,
                             cudaMemcpyDeviceToDevice, as_stream(stream)));
    return A2A_OK;
}

int a2a_export_dispatch(a2a_ctx* c, int32_t* counts, void* rows, int32_t* meta, void* stream) {
    if (c == nullptr || counts == nullptr || rows == nullptr || meta == nullptr) return A2A_ERR_CONFIG;
    if (!c->sent) return A2A_ERR_STATE;
    DeviceGuard guard(c->cfg.device);
    export_dispatch_kernel<<<c->num_sms * 2, kThreads, 0, as_stream(stream)>>>(call_params(c), counts,
                                                                              static_cast<uint4*>(rows), meta);
    c->launches++;
    CUDA_TRY(cudaGetLastError());
    return A2A_OK;
}

int a2a_expert_buffers(a2a_ctx* c, void** rows, int32_t** counts) {
    if (c == nullptr) return A2A_ERR_CONFIG;
    if (rows) *rows = c->region + c->lay.off_rows;
    if (counts) *counts = reinterpret_cast<int32_t*>(c->region + c->lay.off_counts);
    return A2A_OK;
}

int a2a_route_buffers(a2a_ctx* c, int32_t** slots, int32_t** send_counts) {
    if (c == nullptr) return A2A_ERR_CONFIG;
    if (slots) *slots = c->p.slot;
    if (send_counts) *send_counts = c->p.send_counts;
    return A2A_OK;
}

int a2a_copy_route(a2a_ctx* c, int32_t* slots_out, int32_t* send_counts_out, void* stream) {
    if (c == nullptr) return A2A_ERR_CONFIG;
    if (!c->routed) return A2A_ERR_STATE;
    DeviceGuard guard(c->cfg.device);
    const size_t pairs = (size_t)c->cur_tokens * c->cfg.experts_per_token;
    if (slots_out && pairs)
        CUDA_TRY(cudaMemcpyAsync(slots_out, c->p.slot, pairs * 4, cudaMemcpyDeviceToDevice, as_stream(stream)));
    if (send_counts_out)
        CUDA_TRY(cudaMemcpyAsync(send_counts_out, c->p.send_counts, (size_t)c->cfg.num_experts * 4,
                                 cudaMemcpyDeviceToDevice, as_stream(stream)));
    return A2A_OK;
}

int a2a_trace_enable(a2a_ctx* c, int on) {
    if (c == nullptr) return A2A_ERR_CONFIG;
    DeviceGuard guard(c->cfg.device);
    CUDA_TRY(cudaDeviceSynchronize());
    if (on) CUDA_TRY(cudaMemset(c->trace, 0, (size_t)kTraceBlocks * kNumStamps * 8));
    c->p.trace = on ? c->trace : nullptr;
    return A2A_OK;
}

int a2a_trace_read(a2a_ctx* c, int64_t* out, int max_blocks, int* blocks, int* stamps_per_block) {
    if (c == nullptr || out == nullptr || max_blocks < 0) return A2A_ERR_CONFIG;
    DeviceGuard guard(c->cfg.device);
    CUDA_TRY(cudaDeviceSynchronize());
    int n = c->last_grid < max_blocks ? c->last_grid : max_blocks;
    if (n > 0) CUDA_TRY(cudaMemcpy(out, c->trace, (size_t)n * kNumStamps * 8, cudaMemcpyDeviceToHost));
    if (blocks) *blocks = n;
    if (stamps_per_block) *stamps_per_block = kNumStamps;
    return A2A_OK;
}

int a2a_status(a2a_ctx* c, a2a_status_t* out) {
    if (c == nullptr || out == nullptr) return A2A_ERR_CONFIG;
    DeviceGuard guard(c->cfg.device);
    CUDA_TRY(cudaMemcpyAsync(out, c->p.status, sizeof(*out), cudaMemcpyDeviceToHost, c->side));
    CUDA_TRY(cudaStreamSynchronize(c->side));
    return A2A_OK;
}

int a2a_status_peek(a2a_ctx* c) { return c ? *reinterpret_cast<volatile int*>(c->host_code) : A2A_ERR_CONFIG; }

int a2a_status_clear(a2a_ctx* c) {
    if (c == nullptr) return A2A_ERR_CONFIG;
    DeviceGuard guard(c->cfg.device);
    CUDA_TRY(cudaDeviceSynchronize());
    CUDA_TRY(cudaMemset(c->p.status, 0, sizeof(a2a_status_t)));
    *reinterpret_cast<volatile int*>(c->host_code) = 0;
    CUDA_TRY(cudaMemset(c->p.tickets, 0, 8 * sizeof(uint32_t)));
    CUDA_TRY(cudaMemset(c->p.ptickets, 0, 2 * A2A_MAX_WORLD * sizeof(uint32_t)));
    return A2A_OK;
}

int64_t a2a_launch_count(a2a_ctx* c) { return c ? c->launches : 0; }

size_t a2a_symmetric_bytes(a2a_ctx* c) { return c ? c->lay.total : 0; }

}  // extern "C"
