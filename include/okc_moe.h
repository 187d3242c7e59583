/*
 * okc_moe.h — C ABI of the B200 (sm_100a) NVFP4 W4A16 MoE decode step.
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, allocates no memory
 * (okc_moe_experts_profiled alone creates and destroys CUDA events), enqueues its work on the
 * given CUDA stream and returns 0 or a negative okc_moe_error.  All device buffers are owned by the caller.
 * Device-side waits are bounded; a wait that ran out is reported through the status
 * word (okc_moe_read_status), never by a trap.
 *
 * The calls replace, in the reference (tech-cosmos/okc-muse-kernels), the `moe_*_launch`
 * host wrappers that `muse_moe_w4a16/submission.py` binds through
 * torch.utils.cpp_extension.load_inline (submission.py:5812-5859) and that its
 * `prepare` / `kernel_fn` call (submission.py:6011, 6518).
 */
#ifndef OKC_MOE_H
#define OKC_MOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* okc_stream_t; /* a cudaStream_t */

enum okc_moe_error {
  OKC_OK = 0,
  OKC_ERR_BAD_PLAN = -1,     /* shape not supported (see okc_moe_plan) */
  OKC_ERR_BAD_ARG = -2,      /* null pointer, misaligned pointer, T out of range */
  OKC_ERR_CUDA = -3,         /* a CUDA runtime / driver call failed */
  OKC_ERR_NO_DEVICE = -4,    /* no sm_100 device is current */
  OKC_ERR_TIMEOUT = -5,      /* status word: a bounded device wait ran out */
  OKC_ERR_TOO_LARGE = -6     /* size beyond a fixed capacity */
};

/*
 * Shape of one MoE layer shard.  Mirrors the `config` dict of the reference's inputs
 * (muse_moe_w4a16/reference.py:83-84: d_hidden, d_expert, n_experts, local_start,
 * local_count, top_k) plus what the reference hard-codes (post-expert norm on/off)
 * and what it lacks (a shared expert).
 * Limits: hidden % 256 == 0, inter % 256 == 0, n_experts <= 512, top_k <= 16,
 * 1 <= max_tokens <= 4096, shared_inter == 0 or == inter.
 */
typedef struct okc_moe_plan {
  int32_t hidden;        /* H: model width of the MoE block */
  int32_t inter;         /* I: expert intermediate width */
  int32_t n_experts;     /* E: experts in the whole layer (router width) */
  int32_t top_k;         /* experts per token */
  int32_t local_start;   /* first expert held by this GPU */
  int32_t local_count;   /* experts held by this GPU */
  int32_t shared_inter;  /* 0, or the shared expert's intermediate width (== inter) */
  int32_t max_tokens;    /* capacity the workspace is sized for */
  int32_t post_norm;     /* 1: per-route RMSNorm(y*(1+w), eps 1e-8) before weighting (reference.py:88-90) */
  int32_t reserved[7];   /* must be zero */
} okc_moe_plan;

typedef struct okc_moe_sizes {
  uint64_t packed_w13_bytes;   /* repacked w13 of (local_count + shared) experts */
  uint64_t packed_w2_bytes;    /* repacked w2 of the same experts */
  uint64_t workspace_bytes;    /* scratch for one step in flight; zeroed once by the caller before its first step
                                  (the control words at its start count and hand over between kernels) */
  uint32_t expert_slots;       /* local_count + (shared_inter ? 1 : 0) */
  uint32_t routes_per_token;   /* top_k + (shared_inter ? 1 : 0) */
} okc_moe_sizes;

/* Library / format version (major*100 + minor). */
int okc_moe_version(void);
const char* okc_moe_strerror(int code);

/* Sizes of the caller-owned buffers for a plan.  Replaces the `torch.empty` sizes computed in
 * `prepare` and `kernel_fn` (submission.py:6011-6070, 6527-6531). */
int okc_moe_query(const okc_moe_plan* plan, okc_moe_sizes* out);

/*
 * Lossless repack of `count` experts' NVFP4 tensors into stage images, written at expert slot
 * `first_slot` of packed_w13 / packed_w2.  w13: uint8 [count, 2I, H/2], w13_sf: e4m3 bytes
 * [count, 2I, H/16], w2: uint8 [count, H, I/2], w2_sf: [count, H, I/16] (device pointers to the
 * first expert to repack).  Replaces `_pack_weight` / `_pack_scales` / `_sq_pack`
 * (submission.py:5916-5952).
 */
int okc_moe_repack(const okc_moe_plan* plan, const void* w13, const void* w13_sf, const void* w2,
                   const void* w2_sf, int first_slot, int count, void* packed_w13, void* packed_w2,
                   okc_stream_t stream);

/*
 * Router + token->expert sort.  logits: f32 [T, E] (row stride E).  Writes ids int32 [T, top_k]
 * (global expert ids, descending logit, ties to the lowest index) and weights f32 [T, top_k]
 * (softmax over the selected logits), and the sorted route tables inside `workspace`.
 * Tokens [own_t0, own_t1) also get a route to the shared expert when the plan has one.
 * Replaces `_routing` (muse_decode_layer/layer.py:374-414) and `moe_route` / `moe_routegather`
 * (submission.py:324-368, 2236-2328).
 */
int okc_moe_route(const okc_moe_plan* plan, const float* logits, int T, int own_t0, int own_t1,
                  int32_t* ids, float* weights, void* workspace, okc_stream_t stream);

/* The sort alone, for callers that bring their own routing (the reference's `kernel_fn` inputs
 * `topk_ids` / `topk_weights`, submission.py:23-48).  ids outside the local range are skipped. */
int okc_moe_sort(const okc_moe_plan* plan, const int32_t* ids, const float* weights, int T,
                 int own_t0, int own_t1, void* workspace, okc_stream_t stream);

/*
 * The router of the reference's decode layer, fused with the step before it: the router logits
 * `hidden . w^T` are computed from the token rows (FP32 multiply-adds, split over K; they never exist
 * as a tensor) and go straight into the top-k.  Replaces `_router_split` + `_routing`
 * (muse_decode_layer/layer.py:325-351, 374-414) and `route` (muse_decode_layer/reference.py:419-424).
 *   mode 0: softmax top-k as okc_moe_route.
 *   mode 1: scores = sigmoid(multiplier * logit); the top_k of scores + bias are chosen (ties to the
 *           lowest id); weights = chosen scores / (their sum + 1e-15).
 * w: f32 [E, H], or w_split (see okc_router), or neither: take `logits` f32 [T, E] instead and only apply the
 * mode; bias: f32 [E] or NULL.
 * With w / w_split: T <= 256, E a multiple of 16; the per-route output area of `workspace` is used as scratch.
 * Then sorts the routes as okc_moe_route does.
 */
typedef struct okc_router {
  const float* w;
  const float* bias;
  int32_t mode;
  float multiplier;
  const void* w_split;   /* instead of w: the router matrix as bf16 hi + lo rows [2 E, H] (okc_moe_router_split);
                            the logits are then computed on the tensor cores, two bf16 MMAs per K step */
} okc_router;
/* w f32 [E, H] -> w_split bf16 [2 E, H]: rows [0, E) = bf16(w), rows [E, 2 E) = bf16(w - bf16(w)); once per router
 * matrix.  Replaces the split in `_router_split` (muse_decode_layer/layer.py:325-351). */
int okc_moe_router_split(const float* w, int n_experts, int hidden, void* w_split, okc_stream_t stream);
int okc_moe_route_hidden(const okc_moe_plan* plan, const okc_router* router, const void* hidden,
                         int64_t hidden_stride, const float* logits, int T, int own_t0, int own_t1,
                         int32_t* ids, float* weights, void* workspace, okc_stream_t stream);

/*
 * The experts on the routes sorted into `workspace`: gather -> one persistent launch of the
 * gate_up GEMM + SiLU*mul units and the down GEMM (x routing weight, un-permuted) units, a down
 * unit starting as soon as the gate_up units of its own work item are done -> per-token combine.
 * hidden: bf16 [T, H] with row stride `hidden_stride` elements.  gs13 / gs2: f32 [expert_slots].
 * post_norm_w: bf16 [H] or NULL.  out: bf16 [T, H] when out_f32 == 0, else f32 [T, H] (the
 * partial sum an expert-parallel reduce-scatter consumes).  Rows with no local route are zero.
 * Replaces `moe_tk2f_launch` / `moe_twm_launch` + `moe_norm*_launch` (submission.py:5453, 5751).
 */
int okc_moe_experts(const okc_moe_plan* plan, const void* packed_w13, const void* packed_w2,
                    const float* gs13, const float* gs2, const void* hidden, int64_t hidden_stride,
                    int T, const void* post_norm_w, void* workspace, void* out, int out_f32,
                    okc_stream_t stream);

/*
 * okc_moe_experts with the pre-expert RMSNorm of the reference's decode layer applied while the token
 * rows are gathered: a row x becomes bf16(x * rsqrt(mean(x^2) + pre_eps) * pre_gain[k]) before the gate_up
 * GEMM (the layer passes pre_gain = 1 + pre_expert_norm, eps 1e-5).  hidden: bf16 rows, or with
 * hidden_f32 != 0 f32 rows, which are rounded to bf16 first as the reference does (the pooler's FP32
 * output goes in without a round trip); hidden_stride in elements of that type.  pre_gain: f32 [H],
 * H <= 8192.  Together with out_f32 = 1 (FP32 rows for the unpooler) these are the steps either side of
 * the MoE block in the layer.  Replaces `moe_gathern_launch` (muse_decode_layer/layer.py:1700-1745).
 */
int okc_moe_experts_prenorm(const okc_moe_plan* plan, const void* packed_w13, const void* packed_w2,
                            const float* gs13, const float* gs2, const void* hidden, int64_t hidden_stride,
                            int hidden_f32, const float* pre_gain, float pre_eps, int T,
                            const void* post_norm_w, void* workspace, void* out, int out_f32,
                            okc_stream_t stream);

/* okc_moe_experts with CUDA events around its three kernels: synchronises, then writes their
 * durations in milliseconds to the host array phase_ms[4] = {gather, grouped GEMMs (gate_up and
 * down units in one launch), combine, whole call}.
 * A measurement aid (it creates and destroys four events); not for the serving path.  Plays the
 * role of the reference's DIAG timing harness (submission.py:6151-6231). */
int okc_moe_experts_profiled(const okc_moe_plan* plan, const void* packed_w13, const void* packed_w2,
                             const float* gs13, const float* gs2, const void* hidden,
                             int64_t hidden_stride, int T, const void* post_norm_w, void* workspace,
                             void* out, int out_f32, okc_stream_t stream, float* phase_ms);

/* f32 [n] -> bf16 [n] (n % 4 == 0): the cast after an expert-parallel reduce-scatter of FP32
 * partial sums.  The reference has no counterpart (its expert all-reduce is not run,
 * muse_moe_w4a16/baseline.py:8). */
int okc_moe_cast_bf16(const float* in, void* out_bf16, int64_t n, okc_stream_t stream);

/* okc_moe_route followed by okc_moe_experts. */
int okc_moe_step(const okc_moe_plan* plan, const void* packed_w13, const void* packed_w2,
                 const float* gs13, const float* gs2, const void* hidden, int64_t hidden_stride,
                 const float* logits, int T, int own_t0, int own_t1, const void* post_norm_w,
                 int32_t* ids, float* weights, void* workspace, void* out, int out_f32,
                 okc_stream_t stream);

/*
 * okc_moe_step for callers that cannot give it a workspace because they cannot allocate one.
 * (No counterpart in the reference: its kernel_fn allocates its scratch with torch.empty on
 * every call.)  Think of a serving process that claimed all device memory for its own pool at
 * start-up, a plugin living inside such a process, or any caller for which cudaMalloc is off
 * limits while it runs.  The scratch of the step is a fixed array of
 * OKC_MOE_STATIC_SCRATCH_BYTES built into the library; each GPU that loads the library holds it
 * until the process ends.  The call allocates nothing and frees nothing.
 *
 *  - Limit: the plan's workspace_bytes (okc_moe_query; it grows with max_tokens) must not exceed
 *    OKC_MOE_STATIC_SCRATCH_BYTES, otherwise OKC_ERR_TOO_LARGE is returned and nothing runs.
 *    Configuration 2 (H=4096, I=1536, top-8) fits up to max_tokens = 128.
 *  - The first call on each device looks up the array's device address (the device must be
 *    current).  Make that first call before starting any stream capture.
 *  - All calls on a device share the one array.  The call clears the few control words that must
 *    start at zero; everything else is overwritten by the step.  Two calls whose kernels overlap
 *    on the GPU (different streams, or a graph replay racing a direct call) corrupt each other:
 *    keep them on one stream or otherwise serialised.
 *  - The status word of this variant lives in the array, so okc_moe_read_status cannot reach it:
 *    okc_moe_read_status_static reads it (before the next call of this entry point, which clears it).
 * All other arguments are those of okc_moe_step.
 */
#define OKC_MOE_STATIC_SCRATCH_BYTES (32u << 20)
int okc_moe_step_static_scratch(const okc_moe_plan* plan, const void* packed_w13, const void* packed_w2,
                                const float* gs13, const float* gs2, const void* hidden,
                                int64_t hidden_stride, const float* logits, int T, int own_t0, int own_t1,
                                const void* post_norm_w, int32_t* ids, float* weights, void* out,
                                int out_f32, okc_stream_t stream);

/* okc_moe_read_status for the array of okc_moe_step_static_scratch on the current device:
 * synchronises `stream`, returns 0 or OKC_ERR_TIMEOUT with *detail naming the wait that ran out.
 * (No counterpart in the reference.) */
int okc_moe_read_status_static(okc_stream_t stream, int32_t* detail);

/*
 * The exchange steps of the expert-parallel layer over peer memory (NVLink / NVSwitch), for one
 * process per GPU.  No counterpart in the reference: its shards never exchange anything (the expert
 * all-reduce is not run, muse_moe_w4a16/baseline.py:8).
 *
 * Every rank owns one exchange buffer of okc_ep_buffer_bytes() bytes, zeroed once before the first
 * step, and maps the buffers of all ranks into its address space (CUDA IPC or any other peer
 * mapping; the caller's business).  Rank r owns token rows [r*T/world, (r+1)*T/world) of the step.
 *  - okc_ep_gather_tokens: stores this rank's rows (hidden bf16 [T/world, hidden_stride], logits f32
 *    [T/world, E]) into every rank's buffer and returns when every rank's rows have arrived here:
 *    afterwards okc_ep_views' hidden_all [T, H] / logits_all [T, E] hold the whole step's tokens.
 *  - the caller then runs okc_moe_step on them with out = okc_ep_views' partial (f32 [T, H], out_f32 = 1).
 *  - okc_ep_reduce_scatter: out_bf16 [T/world, H] = sum over ranks (rank order) of their partial
 *    rows of this rank's tokens, rounded once.
 * All ranks must make the same calls in the same order.  The waits on other ranks are bounded (five
 * seconds, or okc_ep_comm.wait_limit_ms); one that runs out is reported by okc_ep_read_status (OKC_ERR_TIMEOUT, detail 0x100 + rank
 * for the gather, 0x200 + rank for the reduce) and the step's result is then undefined.
 */
#define OKC_EP_MAX_RANKS 16
typedef struct okc_ep_comm {
  int32_t rank, world;
  int32_t tokens;      /* T of the whole step, a multiple of world */
  int32_t hidden;      /* H, a multiple of 256 */
  int32_t n_experts;   /* E, a multiple of 4 */
  int32_t wait_limit_ms; /* limit of every wait on another rank in milliseconds; 0 = five seconds */
  int32_t reserved[2];   /* must be zero */
  void* peer[OKC_EP_MAX_RANKS]; /* this process's address of rank r's buffer; peer[rank] is its own */
} okc_ep_comm;

uint64_t okc_ep_buffer_bytes(int32_t tokens, int32_t hidden, int32_t n_experts);
int okc_ep_views(const okc_ep_comm* comm, void** hidden_all, void** logits_all, void** partial);
int okc_ep_gather_tokens(const okc_ep_comm* comm, const void* hidden_own, int64_t hidden_stride,
                         const float* logits_own, okc_stream_t stream);
int okc_ep_reduce_scatter(const okc_ep_comm* comm, void* out_bf16, okc_stream_t stream);
/* okc_moe_experts for one rank of the expert-parallel layer with its last kernel replaced: the
 * per-token combine and okc_ep_reduce_scatter in one kernel (a rank's partial sums of its own rows
 * stay in registers).  hidden = okc_ep_views' hidden_all, T = comm->tokens; plans with post_norm are
 * refused (OKC_ERR_BAD_PLAN: use okc_moe_experts + okc_ep_reduce_scatter).  Detail of a wait that
 * ran out: 0x300 + rank. */
int okc_moe_experts_ep(const okc_moe_plan* plan, const void* packed_w13, const void* packed_w2,
                       const float* gs13, const float* gs2, const void* hidden, int64_t hidden_stride,
                       int T, void* workspace, const okc_ep_comm* comm, void* out_bf16,
                       okc_stream_t stream);
/* okc_ep_gather_tokens with the router in it, in one kernel: the rank routes its own token block (softmax
 * top-k, as okc_moe_route) while it stores the rows into every rank's buffer, sends the k ids and weights of
 * each token instead of its logits (they take the place of the logits in the buffer: ids int32 [T, top_k],
 * then weights f32 [T, top_k]; okc_ep_routed_views gives their addresses; needs 2 * top_k <= n_experts), and
 * once every rank's flag has been seen sorts the routes of the whole step into `workspace` as okc_moe_sort
 * does, the shared expert on the rank's own token block.  The caller goes on with okc_moe_experts_ep (or
 * okc_moe_experts + okc_ep_reduce_scatter).  Three launches fewer than gather + route.  No counterpart in the
 * reference. */
int okc_ep_route_gather(const okc_moe_plan* plan, const okc_ep_comm* comm, const void* hidden_own,
                        int64_t hidden_stride, const float* logits_own, void* workspace, okc_stream_t stream);
int okc_ep_routed_views(const okc_ep_comm* comm, int top_k, void** ids_all, void** weights_all);
/* Raises, in this rank's own buffer, the flag that rank `from_rank` raises when its token rows
 * (which = 0) or its partial sums (which = 1) of the coming exchange are in place.  For a harness that
 * runs the ranks of a step one after the other on one device (there the later rank's data is put in
 * place by other means, and a kernel must never wait for a kernel launched after it).  No counterpart
 * in the reference. */
int okc_ep_mark_arrived(const okc_ep_comm* comm, int which, int from_rank, okc_stream_t stream);
/* Synchronises `stream`; returns the status kept in this rank's buffer and clears it. */
int okc_ep_read_status(const okc_ep_comm* comm, okc_stream_t stream, int32_t* detail);

/* Copies the sorted-route tables out of `workspace` for inspection (host or device pointers are
 * NOT interchangeable: all four are device pointers; any may be NULL).  counts: int32
 * [expert_slots]; sorted: int32 [T*routes_per_token] (route index t*routes_per_token+slot per
 * position, -1 padded); pos: int32 [T*routes_per_token]; items: int32 [1 + 4*max_items]
 * (n_items, then (slot, first position, rows, padded rows) per work item.  While no expert has more
 * than 32 rows, experts are cut into items of <= 16 rows when T <= 64 or T * top_k <= 8 * n_experts, else
 * of <= 32 rows; otherwise an expert with up to 16 rows is one item and every other one is cut into items of
 * <= 64 rows.  Padded rows are 16, 32 or 64). */
int okc_moe_export_sort(const okc_moe_plan* plan, const void* workspace, int T, int32_t* counts,
                        int32_t* sorted, int32_t* pos, int32_t* items, int max_items,
                        okc_stream_t stream);

/* Dequantises one repacked matrix back to bf16 [rows, K] scaled by 2^-8 (the factor the GEMM
 * epilogues fold into the global scale): which = 0 for w13 (rows = 2I, K = H), 1 for w2
 * (rows = H, K = I).  A check of the repack + dequantisation arithmetic on CUDA cores. */
int okc_moe_unpack_bf16(const okc_moe_plan* plan, const void* packed, int which, int slot,
                        void* out_bf16, okc_stream_t stream);

/* Synchronises `stream` and returns the step status kept in `workspace`: 0, or
 * OKC_ERR_TIMEOUT with *detail = a code naming the wait that ran out. */
int okc_moe_read_status(const void* workspace, okc_stream_t stream, int32_t* detail);

/* Failure-detection self test: launches one warp that waits, with a short limit, on a barrier
 * nothing will ever complete.  The wait runs out, the kernel returns normally and sets the status
 * words of `workspace` the way a GEMM kernel whose wait ran out does: okc_moe_read_status then
 * returns OKC_ERR_TIMEOUT with detail 0x7e.  The next okc_moe_route / okc_moe_sort call clears
 * the status.  The reference's waits are unbounded spins (submission.py:3862-3869, 394-398). */
int okc_moe_probe_wait_timeout(void* workspace, okc_stream_t stream);

/* Kernels launched by okc_moe_step for a step of more than 32 tokens (top-k, sort, gather, the GEMM launch,
 * combine); up to 32 tokens top-k and sort are one kernel. */
int okc_moe_launches_per_step(void);

#ifdef __cplusplus
}
#endif
#endif /* OKC_MOE_H */
