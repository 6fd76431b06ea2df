/*
 * a2a.h -- C ABI of liba2a.so: MoE all-to-all dispatch / expert placeholder /
 * combine for NVIDIA B200 (sm_100a) over NVLink peer memory.
 *
 * One context per process and GPU ("rank").  Every rank owns one symmetric
 * region of device memory (receive rows, row metadata, per-source counts,
 * epoch flags); peers map it through CUDA IPC (or, inside one process, by
 * pointer).  All data-path functions only enqueue kernels on the caller's
 * stream and never synchronise with the host; they must be called by all ranks
 * collectively, the same number of times, in the same order.
 *
 * Conventions: every function returns an int status -- 0 on success, a positive
 * A2A_ERR_* code for errors detected by this library, or the negated
 * cudaError_t for a CUDA runtime failure.  Device pointers are plain `void*`
 * owned by the caller; `stream` is a cudaStream_t passed as `void*` (NULL =
 * legacy default stream).  A context is not thread-safe.
 *
 * Each entry point cites the interface of the reference
 * (gau-nernst/gpu-mode-kernels, amd-distributed/all2all) that it replaces.
 */
#ifndef A2A_H_
#define A2A_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct a2a_ctx a2a_ctx;

enum {
    A2A_OK = 0,
    A2A_ERR_CONFIG = 1,   /* invalid configuration or argument                          */
    A2A_ERR_CAPACITY = 2, /* a (source, expert) slab would overflow max_num_tokens rows  */
    A2A_ERR_TIMEOUT = 3,  /* a bounded device-side wait on a peer's flag ran out         */
    A2A_ERR_STATE = 4,    /* call order violated (peers not attached, route missing...)  */
    A2A_ERR_ROUTING = 5   /* an expert index outside [0, num_experts), or repeated inside a token */
};

enum { A2A_DTYPE_BF16 = 0, A2A_DTYPE_FP16 = 1 };

/* How dispatch moves token rows to the expert ranks. */
enum {
    A2A_PAYLOAD_DIRECT = 0, /* one row per (token, k), stored straight into the expert's slab     */
    A2A_PAYLOAD_DEDUP = 1,  /* one row per (token, destination rank); the receiver fans it out    */
    A2A_PAYLOAD_FP8 = 2     /* as DEDUP, row quantised to e4m3 with one fp32 scale per 128 values */
};

/* How the one-call forward is scheduled on the GPU. */
enum {
    A2A_SCHEDULE_PHASED = 0,    /* routing, sending, expert pass and combine one after the other      */
    A2A_SCHEDULE_PIPELINED = 1  /* blocks with fixed roles (senders driving the copy engine, routers,
                                   experts, watchers) run the phases concurrently, per peer; needs the
                                   DEDUP or FP8 payload and a device with cooperative launch         */
};

/* How expert outputs get back to the token's rank. */
enum {
    A2A_COMBINE_PULL = 0, /* the home rank pulls each (token, k) row from the expert's slab over NVLink
                             and reduces the K rows with the token's weights (fp32, k ascending)       */
    A2A_COMBINE_PUSH = 1  /* the expert rank reduces the rows of a token that IT holds with the token's
                             weights (fp32) and pushes one partial row per (token, expert rank) home;
                             the home rank adds the partial rows (fp32, rank ascending).  One extra
                             rounding to the element type per partial row; pipelined schedule only.  */
};

enum { A2A_MAX_WORLD = 8, A2A_MAX_EXPERTS = 1024, A2A_MAX_TOPK = 32 };

/* Problem description; the fields of the reference's MoEConfig (reference.py:10-17)
 * plus the rank layout custom_kernel receives in its data tuple (reference.py:253). */
typedef struct a2a_config {
    int32_t rank;            /* this process' rank, 0 <= rank < world_size                   */
    int32_t world_size;      /* 1..A2A_MAX_WORLD; num_experts % world_size == 0              */
    int32_t device;          /* CUDA device ordinal of this rank                             */
    int32_t num_experts;     /* E <= A2A_MAX_EXPERTS; expert e lives on rank e / (E/world)   */
    int32_t experts_per_token; /* K <= A2A_MAX_TOPK, distinct experts per token              */
    int32_t hidden_dim;      /* H, multiple of 8 (of 128 for A2A_PAYLOAD_FP8)                */
    int32_t max_num_tokens;  /* upper bound of tokens per rank and call                      */
    int32_t dtype;           /* A2A_DTYPE_*: element type of x and of the output             */
    int32_t payload;         /* A2A_PAYLOAD_*                                                */
    int32_t timeout_ms;      /* budget of every device-side wait; <= 0 selects 2000 ms       */
    int32_t schedule;        /* A2A_SCHEDULE_*                                               */
    int32_t combine;         /* A2A_COMBINE_* (PUSH needs the pipelined schedule)            */
    int32_t chunks;          /* phased schedule: token chunks a call is pipelined in, 1..4;
                                0 selects 1.  Every rank of a group must pass the same value */
    int32_t senders;         /* pipelined schedule: blocks that only move rows; 0 selects 48
                                (96 at 8 ranks and with the FP8 payload)                     */
} a2a_config;

/* First error recorded by a kernel since the last a2a_status_clear(). */
typedef struct a2a_status_t {
    int32_t code;    /* A2A_OK or A2A_ERR_*                         */
    int32_t rank;    /* rank that recorded it                       */
    int32_t peer;    /* peer rank waited for, or -1                 */
    int32_t phase;   /* 1 route, 2 dispatch-send, 3 dispatch-recv, 4 expert, 5 combine, 6 barrier */
    uint32_t epoch;  /* call number the kernel belonged to          */
    int32_t detail;  /* offending expert index / count / token      */
} a2a_status_t;

const char* a2a_strerror(int status);

/* Text describing the last A2A_ERR_CONFIG a2a_open_peers / a2a_attach_local_peers returned for
 * this context (which rank disagreed, or how many bytes were missing).  Replaces the message of
 * the TORCH_CHECK that guards the reference's IPC set-up (submission_v9.py:33-37, :68-75). */
const char* a2a_last_error(a2a_ctx* ctx);

/* Validate `cfg`, select the device, allocate the symmetric region and the
 * local scratch once (nothing is allocated or zeroed on the data path).
 * Replaces P2PState.__init__ + p2p_state_init (submission_v9.py:881-911, :109-131). */
int a2a_create(a2a_ctx** out, const a2a_config* cfg);

/* Wait for this rank's device work, unmap peers, free everything.  The caller
 * must make sure (host barrier) that no peer still reads this rank's memory.
 * Replaces P2PState.close + p2p_state_destroy (submission_v9.py:913-919, :133-145). */
int a2a_destroy(a2a_ctx* ctx);

/* Size of one exported handle blob: the CUDA IPC handle followed by a fingerprint of the
 * configuration (world size, problem sizes, element type, payload, schedule, combine mode,
 * chunk count, size of the symmetric region).  Replaces the fixed 64 in get_ipc_handle
 * (submission_v9.py:61-66). */
size_t a2a_ipc_handle_bytes(void);

/* Write this rank's handle blob (a2a_ipc_handle_bytes() bytes) to `out` (host
 * memory).  The caller all-gathers the blobs with whatever transport it has
 * (one NCCL or gloo all_gather).  Replaces get_ipc_handle (submission_v9.py:61-66). */
int a2a_export_handle(a2a_ctx* ctx, uint8_t* out);

/* The configuration fingerprint alone (the last 64 bytes of a handle blob) and the check
 * a2a_open_peers applies to the gathered blobs, as pure host functions that need neither a
 * context nor a device: a launcher can refuse a mismatched group before any GPU is touched.
 * a2a_check_handles returns A2A_ERR_CONFIG and describes the problem in `msg` when `nbytes` is not
 * world_size * a2a_ipc_handle_bytes() or when some rank's fingerprint differs from the one `cfg`
 * gives.  No counterpart in the reference (its ranks trust each other's layout). */
int a2a_fingerprint(const a2a_config* cfg, uint8_t* out64);
int a2a_check_handles(const a2a_config* cfg, const uint8_t* all_handles, size_t nbytes, char* msg, size_t msg_len);

/* Map every peer's region from the gathered blobs (`world_size` blobs, rank order,
 * `nbytes` in total).  Nothing is mapped unless the byte count is right and every rank's
 * fingerprint equals this rank's: a truncated gather or a rank created with another payload,
 * schedule or problem size returns A2A_ERR_CONFIG (details: a2a_last_error).  Replaces
 * open_ipc_handle per peer + heap_bases (submission_v9.py:68-75, :898-899). */
int a2a_open_peers(a2a_ctx* ctx, const uint8_t* all_handles, size_t nbytes);

/* Same-process alternative to the two calls above: `peers[r]` is rank r's
 * context living in this process (on this or another GPU).  No counterpart in
 * the reference (it is always one process per GPU); used to run several ranks on
 * one GPU phase by phase, and by single-process multi-GPU callers. */
int a2a_attach_local_peers(a2a_ctx* ctx, a2a_ctx* const* peers);

/* Routing: for every (token, k) the slot of its row inside the
 * (expert, this source) slab, and per-expert send counts.  `topk_idx` is
 * [num_tokens, K] int32 on the device.  Replaces the Python loop of
 * PyTorchAllToAll.dispatch (reference.py:72-88) / block 0 of the v9 send kernel
 * (submission_v9.py:272-312). */
int a2a_route(a2a_ctx* ctx, const int32_t* topk_idx, int num_tokens, void* stream);

/* Dispatch, sending half: push this rank's rows (x is [num_tokens, H], device)
 * into the expert ranks' slabs, then publish counts and a release flag to every
 * peer.  Never waits.  Needs a2a_route of the same call first.  Replaces the
 * exchange of PyTorchAllToAll.dispatch (reference.py:90-120) / dispatch_kernel
 * with DO_SEND (submission_v9.py:313-357). */
int a2a_dispatch_send(a2a_ctx* ctx, const void* x, void* stream);

/* Dispatch, receiving half: wait (bounded) until every source's rows of this
 * call have landed; afterwards the slabs and counts are valid (for
 * DEDUP/FP8 payloads this is also where rows are fanned out / dequantised).
 * Replaces the regroup loop (reference.py:123-148) / dispatch_kernel with
 * DO_RECV (submission_v9.py:365-424). */
int a2a_dispatch_recv(a2a_ctx* ctx, void* stream);

/* The reference's placeholder expert op on the valid received rows, in place:
 * row = dtype(float(row) * (1 + rank)); then tell every home rank its outputs
 * are ready.  Replaces reference.py:262 / fake_moe_kernel (submission_v6.py:381-446). */
int a2a_expert_placeholder(a2a_ctx* ctx, void* stream);

/* a2a_dispatch_recv and a2a_expert_placeholder fused into one kernel (wait, scale
 * the rows as they are found valid, publish); the launch a2a_forward makes.
 * Replaces the same reference lines as those two. */
int a2a_dispatch_recv_expert(a2a_ctx* ctx, void* stream);

/* Variant for a real expert op: the caller has overwritten the rows in place
 * with its own kernel on `stream`; only publish readiness to the home ranks. */
int a2a_expert_done(a2a_ctx* ctx, void* stream);

/* Combine: wait (bounded) for the expert ranks, pull the K expert outputs of
 * each token from the peers and write y[t] = dtype(sum_k float(row_k) * w[t,k])
 * (fp32 accumulation, k ascending).  `topk_weights` is [num_tokens, K] fp32,
 * `y` is [num_tokens, H], both on the device.  Replaces PyTorchAllToAll.combine
 * (reference.py:151-234) / combine_kernel (submission_v9.py:480-673). */
int a2a_combine(a2a_ctx* ctx, const float* topk_weights, void* y, void* stream);

/* route + dispatch + expert placeholder + combine in one call; what
 * custom_kernel(data) runs.  Replaces torch.ops.p2p_module.custom_kernel
 * (submission_v9.py:734-831). */
int a2a_forward(a2a_ctx* ctx, const void* x, const int32_t* topk_idx, const float* topk_weights,
                void* y, int num_tokens, void* stream);

/* Choose how a2a_forward launches: 1 = the whole path as ONE cooperative kernel
 * (default where the device supports cooperative launch), 0 = one kernel per phase.
 * Same results either way.  No counterpart in the reference. */
int a2a_set_fused(a2a_ctx* ctx, int on);

/* a2a_forward for HOST buffers (pinned for speed): copies x, topk_idx and
 * topk_weights to the device, runs the path, copies y back; all asynchronous
 * on `stream`.  This is the call a host-resident caller of custom_kernel makes. */
int a2a_forward_host(a2a_ctx* ctx, const void* x_host, const int32_t* topk_idx_host,
                     const float* topk_weights_host, void* y_host, int num_tokens, void* stream);

/* The roles of the pipelined one-launch kernel as three separate launches (same device code):
 * role 0 = senders + routers (takes x, topk_idx, topk_weights, y and num_tokens; starts the call),
 * role 1 = dispatch watchers + expert blocks, role 2 = expert-flag watchers + combine; roles 1
 * and 2 take no tensors (NULL / 0): they use what role 0 was given.  For stepping several ranks on one GPU -- a
 * kernel that waits for a peer never shares a GPU with the kernel it waits for -- and for
 * timing the roles apart.  Needs a context created with A2A_SCHEDULE_PIPELINED.  The reference
 * splits its fused call the same way into dispatch and combine ops (submission_v9.py:675-731). */
int a2a_pipe_step(a2a_ctx* ctx, int role, const void* x, const int32_t* topk_idx, const float* topk_weights,
                  void* y, int num_tokens, void* stream);

/* Cross-GPU rendezvous on the device: returns (on the stream) once every rank's
 * stream has reached it.  Bounded wait.  Used to align ranks before timing.
 * Plays the role of dist.barrier() around the timed call (my_eval.py:160-172). */
int a2a_barrier(a2a_ctx* ctx, void* stream);

/* Measurement helper: one asynchronous copy of `bytes` from this rank's slab rows into rank
 * `peer`'s slab rows (both dead between calls), on `stream`.  Timed with events while every
 * rank copies to its neighbour it gives the per-direction peer-copy bandwidth of the box, the
 * measured figure NVLink fractions can be read against.  `bytes` must not exceed the slab
 * region.  The reference quotes its link figures from vendor numbers instead (README.md:28-29). */
int a2a_link_probe(a2a_ctx* ctx, int peer, size_t bytes, void* stream);

/* Test/inspection helper: copy what PyTorchAllToAll.dispatch returns
 * (reference.py:148) into caller-provided device buffers:
 * counts [L] int32, rows [L, max_num_tokens*world, H], meta [L, max_num_tokens*world, 5]
 * int32 (global_expert, src_rank, src_token, src_k, 0); rows of one expert ordered by
 * (src_rank, token, k) like the reference.  Padding is left untouched. */
int a2a_export_dispatch(a2a_ctx* ctx, int32_t* counts, void* rows, int32_t* meta, void* stream);

/* Device pointers into this rank's own state (valid until a2a_destroy):
 * the slab rows [L][world][max_num_tokens][H] and the row counts [world][4][L] --
 * cumulative over the (up to 4) token chunks of a call, so with the default single chunk
 * counts[s][0][l] is the number of valid rows of slab (l, s); the layout contract a real
 * expert kernel would consume. */
int a2a_expert_buffers(a2a_ctx* ctx, void** rows, int32_t** counts_by_source);

/* Per-(token,k) slot table [num_tokens*K] int32 and per-expert send counts
 * [num_experts] int32 computed by the last a2a_route (device pointers). */
int a2a_route_buffers(a2a_ctx* ctx, int32_t** slots, int32_t** send_counts);

/* Test/inspection helper: copy those two tables into caller device buffers
 * ([num_tokens*K] and [num_experts] int32) on `stream`. */
int a2a_copy_route(a2a_ctx* ctx, int32_t* slots_out, int32_t* send_counts_out, void* stream);

/* Routing tables without any allocation, for callers that cannot call cudaMalloc where
 * they need them (hosts whose memory pool owns the device, plugins barred from the
 * allocator after start-up, loops that cannot afford a synchronising allocation).  It has
 * no counterpart in the reference, whose state is always allocated up front.  Needs no
 * context; runs on the CURRENT device; writes slots_out [num_tokens * experts_per_token]
 * and send_counts_out [num_experts] (device memory of the caller) with the same values
 * a2a_route + a2a_copy_route give.  Its working tables are a 1 MiB static device array
 * held by every GPU that loads the library.  Limits: num_experts <= 1024, num_tokens <=
 * 4096, experts_per_token <= 32 -- larger requests return A2A_ERR_CONFIG and enqueue
 * nothing.  The first call on a device resolves the array's device address: make it
 * before any stream capture.  All calls on a device share the array (the kernel clears
 * what it uses); calls whose kernels overlap on the GPU race -- keep them ordered.  Unlike
 * a2a_route there is no status word: a pair whose expert index is out of range or repeats an
 * earlier expert of its token is dropped silently -- its slot is -1 and nothing else reports it. */
int a2a_route_noalloc(const int32_t* topk_idx, int num_tokens, int num_experts, int experts_per_token,
                      int32_t* slots_out, int32_t* send_counts_out, void* stream);

/* The reference repository's second task (pmpp_v2/histogram_py): out[b] = number of bytes of
 * data[0..n) equal to b, for b = 0..255 -- torch.bincount(data, minlength=256) on uint8 input
 * (reference.py:6-19; native entry of its submission: submission_v1.py:20-113).  `data` is device
 * memory (any alignment, any n >= 0), `out` 256 int64 in device memory, overwritten.  Needs no
 * context; runs on the current device; enqueues a 2 KB memset and one kernel on `stream`. */
int a2a_histogram256(const uint8_t* data, size_t n, int64_t* out, void* stream);

/* Read the first error recorded by a kernel since the last a2a_status_clear.  Waits for
 * nothing on the caller's streams: reads what is there now. */
int a2a_status(a2a_ctx* ctx, a2a_status_t* out);
/* Forget the recorded error and re-arm the block-arrival counters a cut-short kernel may have
 * left half counted.  REQUIRED after A2A_ERR_TIMEOUT before the context is used again: while a
 * timeout is recorded every wait of every later kernel gives up at once.  Synchronises the device. */
int a2a_status_clear(a2a_ctx* ctx);
/* The code a2a_status would report, read from a word in mapped host memory that the kernels
 * mirror it into: no CUDA call, no synchronisation -- cheap enough to look at before every
 * call (the plugin entry does).  May lag a kernel that is still running.  Plays the role of
 * the exception a failed TORCH_CHECK raises in the reference (submission_v9.py:33-37). */
int a2a_status_peek(a2a_ctx* ctx);

/* In-kernel trace.  While enabled, thread 0 of every block stamps the SM cycle counter
 * at each phase boundary of the launches that follow (slot 0 of a block holds the
 * nanosecond global timer at its start; then start, routed (pipelined: the block's role bits),
 * sent, dispatch-seen, expert-done, expert-seen, combine-done; the pipelined kernel also fills,
 * depending on the block's role, slots 8+i / 16+i with "rows of the i-th source seen / done"
 * (expert blocks), 24+i with "stores to the i-th destination acknowledged" and 8..10 with
 * set-up steps (sender blocks), 24..27 with routing steps (router blocks)).  a2a_trace_read
 * synchronises the device and copies the stamps of the most recent traced launch to host
 * memory: `out` must hold max_blocks * 32 int64 (*stamps_per_block
 * returns the 32).  Both calls synchronise: keep them
 * off the timed path.  Replaces the profile buffer of the final reference submission
 * (submission_v9.py:117, :162-184, p2p_state_get_profile). */
int a2a_trace_enable(a2a_ctx* ctx, int on);
int a2a_trace_read(a2a_ctx* ctx, int64_t* out, int max_blocks, int* blocks, int* stamps_per_block);

/* Number of kernels this context has launched so far. */
int64_t a2a_launch_count(a2a_ctx* ctx);

/* Bytes of the symmetric region / of the local scratch of this context. */
size_t a2a_symmetric_bytes(a2a_ctx* ctx);

#ifdef __cplusplus
}
#endif
#endif /* A2A_H_ */
