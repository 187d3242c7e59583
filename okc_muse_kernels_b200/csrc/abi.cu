// The C ABI declared in include/okc_moe.h: argument checks, tensor-map encoding, launches.
// No allocation, no global mutable state besides the lazily resolved driver entry point.
#include <atomic>
#include <cstdio>
#include <cstring>

#include "format.cuh"
#include "params.cuh"

namespace okc {

// ---- driver entry point for tensor-map encoding (resolved once; the pointer is immutable after)
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static std::atomic<EncodeFn> g_encode{nullptr};

static EncodeFn encode_fn() {
  EncodeFn f = g_encode.load(std::memory_order_acquire);
  if (f) return f;
  void* ptr = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &ptr, 12000, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess || ptr == nullptr)
    return nullptr;
  f = reinterpret_cast<EncodeFn>(ptr);
  g_encode.store(f, std::memory_order_release);
  return f;
}

// bf16 [rows, K] row-major (rows row_stride elements apart; 0: K), box = 64 elements x box_rows, 128-byte swizzle,
// zero fill outside.
static bool encode_rows_map(CUtensorMap* map, void* base, uint64_t rows, uint64_t K, uint32_t box_rows,
                            uint64_t row_stride = 0) {
  EncodeFn f = encode_fn();
  if (!f) return false;
  const cuuint64_t dims[2] = {K, rows};
  const cuuint64_t strides[1] = {(row_stride ? row_stride : K) * 2};
  const cuuint32_t box[2] = {64, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  return f(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static int sm_count() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
  return n;
}

static bool is_sm100() {
  int dev = 0, major = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return false;
  return major == 10;
}

static bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

struct Ws {
  int32_t* meta;
  int32_t* counts;
  int4* items;
  int32_t* done;
  int32_t* sorted;
  int32_t* pos;
  float* wsorted;
  uint16_t* xg;
  uint16_t* inter;
  float* y;
};

static Ws carve(void* workspace, const Geometry& g) {
  uint8_t* b = static_cast<uint8_t*>(workspace);
  Ws w;
  w.meta = reinterpret_cast<int32_t*>(b + g.off_meta);
  w.counts = reinterpret_cast<int32_t*>(b + g.off_counts);
  w.items = reinterpret_cast<int4*>(b + g.off_items);
  w.done = reinterpret_cast<int32_t*>(b + g.off_done);
  w.sorted = reinterpret_cast<int32_t*>(b + g.off_sorted);
  w.pos = reinterpret_cast<int32_t*>(b + g.off_pos);
  w.wsorted = reinterpret_cast<float*>(b + g.off_wsorted);
  w.xg = reinterpret_cast<uint16_t*>(b + g.off_xg);
  w.inter = reinterpret_cast<uint16_t*>(b + g.off_inter);
  w.y = reinterpret_cast<float*>(b + g.off_y);
  return w;
}

// The fields of RouteParams that follow from the plan and the workspace (sources and sinks of ids / weights / logits are left null).
static void fill_route_params(const okc_moe_plan* plan, const Geometry& g, int T, int own_t0, int own_t1, void* workspace,
                              RouteParams& p) {
  Ws w = carve(workspace, g);
  memset(&p, 0, sizeof(p));
  p.meta = w.meta; p.counts = w.counts; p.done = w.done; p.items = w.items; p.sorted = w.sorted; p.pos = w.pos; p.wsorted = w.wsorted;
  p.T = T; p.E = plan->n_experts; p.k = plan->top_k; p.kk = g.kk; p.slots = g.slots;
  p.local_start = plan->local_start; p.local_count = plan->local_count; p.has_shared = plan->shared_inter ? 1 : 0;
  p.own_t0 = own_t0; p.own_t1 = own_t1; p.max_items = g.max_items; p.chunk_rows = chunk_rows_for(T, plan->top_k, plan->n_experts);
  p.router_mode = 0; p.router_mult = 1.0f; p.H = g.H;
}

static int route_common(const okc_moe_plan* plan, const float* logits, const int32_t* ids_in, const float* wts_in,
                        int T, int own_t0, int own_t1, int32_t* ids_out, float* wts_out, void* workspace,
                        cudaStream_t stream, const okc_router* router = nullptr, const void* hidden = nullptr,
                        int64_t hidden_stride = 0) {
  Geometry g;
  if (!plan || !make_geometry(*plan, g)) return OKC_ERR_BAD_PLAN;
  if (!workspace || !aligned(workspace, 256) || T <= 0 || T > plan->max_tokens) return OKC_ERR_BAD_ARG;
  if (own_t0 < 0 || own_t1 < own_t0 || own_t1 > T) return OKC_ERR_BAD_ARG;
  RouteParams p;
  fill_route_params(plan, g, T, own_t0, own_t1, workspace, p);
  p.logits = logits; p.ids_in = ids_in; p.wts_in = wts_in; p.ids_out = ids_out; p.wts_out = wts_out;
  if (router) {
    if (router->mode != 0 && router->mode != 1) return OKC_ERR_BAD_ARG;
    p.router_mode = router->mode; p.router_mult = router->multiplier; p.router_bias = router->bias;
    if (router->w_split) {
      // logits from the token rows on the tensor cores; split-K partial sums in the (not yet used) per-route output area
      if (!hidden || !aligned(hidden, 16) || !aligned(router->w_split, 16) || hidden_stride < g.H || (hidden_stride % 8) != 0)
        return OKC_ERR_BAD_ARG;
      if (T > 256 || (p.E % 16) != 0) return OKC_ERR_BAD_PLAN;
      const int n_kb = g.H / 64, tiles = (p.E + 127) / 128;
      int per = (n_kb + 31) / 32;
      if (per < (tiles * n_kb + 147) / 148) per = (tiles * n_kb + 147) / 148;
      if (per > 3) per = 3;
      if (per < 1) per = 1;
      const long long splits = (n_kb + per - 1) / per;
      const long long room = static_cast<long long>(g.kk) * g.H / p.E;   // [T * kk, H] floats hold `room` arrays [T, E]
      if (splits > room) return OKC_ERR_BAD_PLAN;
      const uint32_t tpad = static_cast<uint32_t>((T + 15) & ~15);
      if (!encode_rows_map(&p.router_wmap, const_cast<void*>(router->w_split), 2ull * p.E, static_cast<uint64_t>(g.H), 128) ||
          !encode_rows_map(&p.router_hmap, const_cast<void*>(hidden), static_cast<uint64_t>(T), static_cast<uint64_t>(g.H), tpad,
                           static_cast<uint64_t>(hidden_stride)))
        return OKC_ERR_CUDA;
      p.router_w_split = static_cast<const uint16_t*>(router->w_split); p.router_kb_per_cta = per;
      p.hidden = static_cast<const uint16_t*>(hidden); p.hidden_stride = hidden_stride;
      p.router_splits = static_cast<int>(splits); p.router_part = carve(workspace, g).y;
    } else if (router->w) {
      // logits from the token rows: split-K partial sums kept in the (not yet used) per-route output area
      if (!hidden || !aligned(hidden, 16) || !aligned(router->w, 16) || hidden_stride < g.H || (hidden_stride % 8) != 0)
        return OKC_ERR_BAD_ARG;
      if (T > 256 || (p.E % 16) != 0) return OKC_ERR_BAD_PLAN;
      long long splits = 148 / (p.E / 16);
      const long long room = static_cast<long long>(g.kk) * g.H / p.E;   // [T * kk, H] floats hold `room` arrays [T, E]
      if (splits > room) splits = room;
      if (splits > g.H / 64) splits = g.H / 64;
      if (splits > 16) splits = 16;
      if (splits < 1) return OKC_ERR_BAD_PLAN;
      p.router_w = router->w; p.hidden = static_cast<const uint16_t*>(hidden); p.hidden_stride = hidden_stride;
      p.router_splits = static_cast<int>(splits); p.router_part = carve(workspace, g).y;
    }
  }
  return launch_route(p, stream) == cudaSuccess ? OKC_OK : OKC_ERR_CUDA;
}

}  // namespace okc

using namespace okc;

extern "C" {

int okc_moe_version(void) { return 101; }

const char* okc_moe_strerror(int code) {
  switch (code) {
    case OKC_OK: return "ok";
    case OKC_ERR_BAD_PLAN: return "plan outside the supported shapes";
    case OKC_ERR_BAD_ARG: return "bad argument (null or misaligned pointer, token count out of range)";
    case OKC_ERR_CUDA: return "a CUDA call failed";
    case OKC_ERR_NO_DEVICE: return "the current device is not an sm_100 GPU";
    case OKC_ERR_TIMEOUT: return "a bounded device-side wait ran out";
    case OKC_ERR_TOO_LARGE: return "size beyond a fixed capacity";
    default: return "unknown error";
  }
}

int okc_moe_launches_per_step(void) { return 5; }   // top-k, sort, gather, GEMMs, combine (top-k + sort are one kernel up to 32 tokens)

int okc_moe_query(const okc_moe_plan* plan, okc_moe_sizes* out) {
  Geometry g;
  if (!plan || !out || !make_geometry(*plan, g)) return OKC_ERR_BAD_PLAN;
  out->packed_w13_bytes = g.w13_expert_bytes * g.slots;
  out->packed_w2_bytes = g.w2_expert_bytes * g.slots;
  out->workspace_bytes = g.total;
  out->expert_slots = static_cast<uint32_t>(g.slots);
  out->routes_per_token = static_cast<uint32_t>(g.kk);
  return OKC_OK;
}

int okc_moe_repack(const okc_moe_plan* plan, const void* w13, const void* w13_sf, const void* w2, const void* w2_sf,
                   int first_slot, int count, void* packed_w13, void* packed_w2, okc_stream_t stream) {
  Geometry g;
  if (!plan || !make_geometry(*plan, g)) return OKC_ERR_BAD_PLAN;
  if (!w13 || !w13_sf || !w2 || !w2_sf || !packed_w13 || !packed_w2) return OKC_ERR_BAD_ARG;
  if (first_slot < 0 || count <= 0 || first_slot + count > g.slots) return OKC_ERR_BAD_ARG;
  if (!aligned(w13, 16) || !aligned(w2, 16) || !aligned(packed_w13, 16) || !aligned(packed_w2, 16)) return OKC_ERR_BAD_ARG;
  RepackParams a;
  a.w = static_cast<const uint8_t*>(w13); a.sf = static_cast<const uint8_t*>(w13_sf);
  a.out = static_cast<uint8_t*>(packed_w13);
  a.rows = 2 * g.I; a.K = g.H; a.pairs = g.pairs13; a.stages = g.stages13; a.first_slot = first_slot; a.count = count;
  a.is_w13 = 1; a.inter = g.I; a.expert_bytes = g.w13_expert_bytes;
  if (launch_repack(a, reinterpret_cast<cudaStream_t>(stream)) != cudaSuccess) return OKC_ERR_CUDA;
  RepackParams b;
  b.w = static_cast<const uint8_t*>(w2); b.sf = static_cast<const uint8_t*>(w2_sf);
  b.out = static_cast<uint8_t*>(packed_w2);
  b.rows = g.H; b.K = g.I; b.pairs = g.pairs2; b.stages = g.stages2; b.first_slot = first_slot; b.count = count;
  b.is_w13 = 0; b.inter = g.I; b.expert_bytes = g.w2_expert_bytes;
  if (launch_repack(b, reinterpret_cast<cudaStream_t>(stream)) != cudaSuccess) return OKC_ERR_CUDA;
  return OKC_OK;
}

int okc_moe_unpack_bf16(const okc_moe_plan* plan, const void* packed, int which, int slot, void* out_bf16,
                        okc_stream_t stream) {
  Geometry g;
  if (!plan || !make_geometry(*plan, g)) return OKC_ERR_BAD_PLAN;
  if (!packed || !out_bf16 || slot < 0 || slot >= g.slots || (which != 0 && which != 1)) return OKC_ERR_BAD_ARG;
  UnpackParams u;
  const size_t eb = which == 0 ? g.w13_expert_bytes : g.w2_expert_bytes;
  u.packed = static_cast<const uint8_t*>(packed) + eb * slot;
  u.out = static_cast<uint16_t*>(out_bf16);
  u.K = which == 0 ? g.H : g.I;
  u.pairs = which == 0 ? g.pairs13 : g.pairs2;
  u.stages = which == 0 ? g.stages13 : g.stages2;
  u.is_w13 = which == 0; u.inter = g.I;
  return launch_unpack(u, reinterpret_cast<cudaStream_t>(stream)) == cudaSuccess ? OKC_OK : OKC_ERR_CUDA;
}

int okc_moe_route(const okc_moe_plan* plan, const float* logits, int T, int own_t0, int own_t1, int32_t* ids,
                  float* weights, void* workspace, okc_stream_t stream) {
  if (!logits || !ids || !weights) return OKC_ERR_BAD_ARG;
  return route_common(plan, logits, nullptr, nullptr, T, own_t0, own_t1, ids, weights, workspace,
                      reinterpret_cast<cudaStream_t>(stream));
}

int okc_moe_router_split(const float* w, int n_experts, int hidden, void* w_split, okc_stream_t stream) {
  if (!w || !w_split || n_experts <= 0 || hidden <= 0 || !aligned(w_split, 16)) return OKC_ERR_BAD_ARG;
  return launch_router_split(w, w_split, static_cast<size_t>(n_experts) * hidden, reinterpret_cast<cudaStream_t>(stream)) == cudaSuccess
             ? OKC_OK : OKC_ERR_CUDA;
}

int okc_moe_sort(const okc_moe_plan* plan, const int32_t* ids, const float* weights, int T, int own_t0, int own_t1,
                 void* workspace, okc_stream_t stream) {
  if (!ids || !weights) return OKC_ERR_BAD_ARG;
  return route_common(plan, nullptr, ids, weights, T, own_t0, own_t1, nullptr, nullptr, workspace,
                      reinterpret_cast<cudaStream_t>(stream));
}

int okc_moe_route_hidden(const okc_moe_plan* plan, const okc_router* router, const void* hidden, int64_t hidden_stride,
                         const float* logits, int T, int own_t0, int own_t1, int32_t* ids, float* weights,
                         void* workspace, okc_stream_t stream) {
  if (!router || !ids || !weights) return OKC_ERR_BAD_ARG;
  if (((router->w != nullptr) + (router->w_split != nullptr) + (logits != nullptr)) != 1) return OKC_ERR_BAD_ARG;   // one source of logits
  if (!is_sm100()) return OKC_ERR_NO_DEVICE;
  return route_common(plan, logits, nullptr, nullptr, T, own_t0, own_t1, ids, weights, workspace,
                      reinterpret_cast<cudaStream_t>(stream), router, hidden, hidden_stride);
}

// Launches the four kernels of the expert phase; `ev`, when given, holds five events recorded
// before / between / after them (gather, gate_up, down, combine).
static bool ep_params(const okc_ep_comm* c, EpParams& p);

// Optional pre-expert norm of the token rows, applied by the gather.
struct PreNorm {
  const float* gain;   // f32 [H]
  float eps;
  int hidden_f32;      // the token rows are f32 (rounded to bf16 first) instead of bf16
};

static int experts_impl(const okc_moe_plan* plan, const void* packed_w13, const void* packed_w2, const float* gs13,
                        const float* gs2, const void* hidden, int64_t hidden_stride, int T, const void* post_norm_w,
                        void* workspace, void* out, int out_f32, cudaStream_t stream, cudaEvent_t* ev,
                        const EpParams* ep = nullptr, const PreNorm* pre = nullptr) {
  Geometry g;
  if (!plan || !make_geometry(*plan, g)) return OKC_ERR_BAD_PLAN;
  if (!packed_w13 || !packed_w2 || !gs13 || !gs2 || !hidden || !workspace || !out) return OKC_ERR_BAD_ARG;
  const bool f32_rows = pre != nullptr && pre->hidden_f32 != 0;
  if (T <= 0 || T > plan->max_tokens || hidden_stride < g.H || (hidden_stride % (f32_rows ? 4 : 8)) != 0) return OKC_ERR_BAD_ARG;
  if (pre && (!pre->gain || !aligned(pre->gain, 16) || !(pre->eps >= 0.0f) || g.H > 8192)) return OKC_ERR_BAD_ARG;
  if (!aligned(packed_w13, 16) || !aligned(packed_w2, 16) || !aligned(hidden, 16) || !aligned(workspace, 256) ||
      !aligned(out, 16))
    return OKC_ERR_BAD_ARG;
  if ((plan->post_norm != 0) != (post_norm_w != nullptr)) return OKC_ERR_BAD_ARG;
  if (post_norm_w && !aligned(post_norm_w, 8)) return OKC_ERR_BAD_ARG;
  if (!is_sm100()) return OKC_ERR_NO_DEVICE;
  const int sms = sm_count();
  if (sms <= 0) return OKC_ERR_CUDA;
  Ws w = carve(workspace, g);
  const int R = T * g.kk;

  // A step of a few tokens needs no gathered copy of its rows: the GEMM's producer fetches each row of a work item
  // from `hidden` itself.  Larger steps (items of up to 64 rows: one boxed copy instead of 64) and steps with the
  // pre-expert norm go through the gather kernel.
  const bool direct = pre == nullptr && T <= kDirectRowsMaxTokens;
  if (ev && cudaEventRecord(ev[0], stream) != cudaSuccess) return OKC_ERR_CUDA;
  if (!direct) {
    const cudaError_t ge = pre ? launch_gather_norm(hidden, hidden_stride, pre->hidden_f32, pre->gain, pre->eps, w.meta, w.sorted,
                                                    g.kk, g.H, R, w.xg, w.done, g.max_items, stream)
                               : launch_gather(hidden, hidden_stride, w.meta, w.sorted, g.kk, g.H, R, w.xg, w.done, g.max_items, stream);
    if (ge != cudaSuccess) return OKC_ERR_CUDA;
  }
  if (ev && cudaEventRecord(ev[1], stream) != cudaSuccess) return OKC_ERR_CUDA;

  // Both GEMM phases in one persistent launch: gate_up units first, then down units, each down
  // unit waiting for the gate_up units of its own work item only.
  MoeGemmParams a;
  memset(&a, 0, sizeof(a));
  const uint32_t boxes[5] = {4, 8, 16, 32, 64};
  for (int i = 0; i < 5; ++i) {
    if (!encode_rows_map(&a.ph[0].bmap[i], w.xg, static_cast<uint64_t>(g.Rpad), static_cast<uint64_t>(g.H), boxes[i])) return OKC_ERR_CUDA;
    if (!encode_rows_map(&a.ph[1].bmap[i], w.inter, static_cast<uint64_t>(g.Rpad), static_cast<uint64_t>(g.I), boxes[i])) return OKC_ERR_CUDA;
  }
  a.ph[0].wpacked = static_cast<const uint8_t*>(packed_w13); a.ph[0].gs = gs13;
  a.ph[0].pairs = g.pairs13; a.ph[0].stages = g.stages13; a.ph[0].expert_bytes = g.w13_expert_bytes;
  a.ph[1].wpacked = static_cast<const uint8_t*>(packed_w2); a.ph[1].gs = gs2;
  a.ph[1].pairs = g.pairs2; a.ph[1].stages = g.stages2; a.ph[1].expert_bytes = g.w2_expert_bytes;
  a.meta = w.meta; a.items = w.items; a.done = w.done;
  a.inter = w.inter; a.I = g.I; a.H = g.H; a.y = w.y; a.sorted = w.sorted; a.wsorted = w.wsorted;
  a.weighted = plan->post_norm ? 0 : 1;
  a.kk = g.kk;
  if (direct) {
    a.direct_rows = 1;
    if (!encode_rows_map(&a.hmap, const_cast<void*>(hidden), static_cast<uint64_t>(T), static_cast<uint64_t>(g.H), 1,
                         static_cast<uint64_t>(hidden_stride)))
      return OKC_ERR_CUDA;
  }
  a.phase_lo = 0; a.phase_hi = 1; a.work_counter = w.meta + kMetaWorkFused;
  if (launch_gemm(a, sms, stream) != cudaSuccess) return OKC_ERR_CUDA;
  if (ev && cudaEventRecord(ev[2], stream) != cudaSuccess) return OKC_ERR_CUDA;

  CombineParams c;
  c.y = w.y; c.pos = w.pos; c.wsorted = w.wsorted; c.post_w = static_cast<const uint16_t*>(post_norm_w);
  c.out = out; c.kk = g.kk; c.H = g.H; c.out_f32 = out_f32 ? 1 : 0;
  c.meta = w.meta; c.done = w.done; c.max_items = g.max_items;
  if (ep) {
    // the combine and the reduce-scatter over the ranks in one kernel
    if (launch_ep_combine_reduce(*ep, c, stream) != cudaSuccess) return OKC_ERR_CUDA;
  } else if (launch_combine(c, T, stream) != cudaSuccess) {
    return OKC_ERR_CUDA;
  }
  if (ev && cudaEventRecord(ev[3], stream) != cudaSuccess) return OKC_ERR_CUDA;
  return OKC_OK;
}

int okc_moe_experts(const okc_moe_plan* plan, const void* packed_w13, const void* packed_w2, const float* gs13,
                    const float* gs2, const void* hidden, int64_t hidden_stride, int T, const void* post_norm_w,
                    void* workspace, void* out, int out_f32, okc_stream_t stream) {
  return experts_impl(plan, packed_w13, packed_w2, gs13, gs2, hidden, hidden_stride, T, post_norm_w, workspace, out,
                      out_f32, reinterpret_cast<cudaStream_t>(stream), nullptr);
}

int okc_moe_experts_prenorm(const okc_moe_plan* plan, const void* packed_w13, const void* packed_w2, const float* gs13,
                            const float* gs2, const void* hidden, int64_t hidden_stride, int hidden_f32,
                            const float* pre_gain, float pre_eps, int T, const void* post_norm_w, void* workspace,
                            void* out, int out_f32, okc_stream_t stream) {
  PreNorm pre;
  pre.gain = pre_gain; pre.eps = pre_eps; pre.hidden_f32 = hidden_f32 ? 1 : 0;
  if (!pre_gain) return OKC_ERR_BAD_ARG;
  return experts_impl(plan, packed_w13, packed_w2, gs13, gs2, hidden, hidden_stride, T, post_norm_w, workspace, out,
                      out_f32, reinterpret_cast<cudaStream_t>(stream), nullptr, nullptr, &pre);
}

int okc_moe_experts_profiled(const okc_moe_plan* plan, const void* packed_w13, const void* packed_w2,
                             const float* gs13, const float* gs2, const void* hidden, int64_t hidden_stride, int T,
                             const void* post_norm_w, void* workspace, void* out, int out_f32, okc_stream_t stream_,
                             float* phase_ms) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (!phase_ms) return OKC_ERR_BAD_ARG;
  cudaEvent_t ev[4];
  int made = 0;
  int rc = OKC_OK;
  for (; made < 4; ++made)
    if (cudaEventCreate(&ev[made]) != cudaSuccess) { rc = OKC_ERR_CUDA; break; }
  if (rc == OKC_OK)
    rc = experts_impl(plan, packed_w13, packed_w2, gs13, gs2, hidden, hidden_stride, T, post_norm_w, workspace, out,
                      out_f32, stream, ev);
  if (rc == OKC_OK && cudaEventSynchronize(ev[3]) != cudaSuccess) rc = OKC_ERR_CUDA;
  if (rc == OKC_OK) {
    for (int i = 0; i < 3; ++i)
      if (cudaEventElapsedTime(&phase_ms[i], ev[i], ev[i + 1]) != cudaSuccess) rc = OKC_ERR_CUDA;
    if (cudaEventElapsedTime(&phase_ms[3], ev[0], ev[3]) != cudaSuccess) rc = OKC_ERR_CUDA;
  }
  for (int i = 0; i < made; ++i) cudaEventDestroy(ev[i]);
  return rc;
}

int okc_moe_cast_bf16(const float* in, void* out_bf16, int64_t n, okc_stream_t stream) {
  if (!in || !out_bf16 || n < 0 || (n % 4) != 0 || !aligned(in, 16) || !aligned(out_bf16, 8)) return OKC_ERR_BAD_ARG;
  if (n == 0) return OKC_OK;
  return launch_cast(in, out_bf16, n, reinterpret_cast<cudaStream_t>(stream)) == cudaSuccess ? OKC_OK : OKC_ERR_CUDA;
}

int okc_moe_step(const okc_moe_plan* plan, const void* packed_w13, const void* packed_w2, const float* gs13,
                 const float* gs2, const void* hidden, int64_t hidden_stride, const float* logits, int T, int own_t0,
                 int own_t1, const void* post_norm_w, int32_t* ids, float* weights, void* workspace, void* out,
                 int out_f32, okc_stream_t stream) {
  int rc = okc_moe_route(plan, logits, T, own_t0, own_t1, ids, weights, workspace, stream);
  if (rc != OKC_OK) return rc;
  return okc_moe_experts(plan, packed_w13, packed_w2, gs13, gs2, hidden, hidden_stride, T, post_norm_w, workspace, out,
                         out_f32, stream);
}

int okc_moe_export_sort(const okc_moe_plan* plan, const void* workspace, int T, int32_t* counts, int32_t* sorted,
                        int32_t* pos, int32_t* items, int max_items, okc_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  Geometry g;
  if (!plan || !make_geometry(*plan, g)) return OKC_ERR_BAD_PLAN;
  if (!workspace || T <= 0 || T > plan->max_tokens) return OKC_ERR_BAD_ARG;
  Ws w = carve(const_cast<void*>(workspace), g);
  const size_t R = static_cast<size_t>(T) * g.kk;
  cudaError_t e = cudaSuccess;
  if (counts && e == cudaSuccess) e = cudaMemcpyAsync(counts, w.counts, sizeof(int32_t) * g.slots, cudaMemcpyDeviceToDevice, stream);
  if (sorted && e == cudaSuccess) e = cudaMemcpyAsync(sorted, w.sorted, sizeof(int32_t) * R, cudaMemcpyDeviceToDevice, stream);
  if (pos && e == cudaSuccess) e = cudaMemcpyAsync(pos, w.pos, sizeof(int32_t) * R, cudaMemcpyDeviceToDevice, stream);
  if (items && e == cudaSuccess) {
    const int n = max_items < g.max_items ? max_items : g.max_items;
    e = cudaMemcpyAsync(items, w.meta + kMetaItems, sizeof(int32_t), cudaMemcpyDeviceToDevice, stream);
    if (e == cudaSuccess && n > 0)
      e = cudaMemcpyAsync(items + 1, w.items, sizeof(int32_t) * 4 * n, cudaMemcpyDeviceToDevice, stream);
  }
  return e == cudaSuccess ? OKC_OK : OKC_ERR_CUDA;
}

int okc_moe_probe_wait_timeout(void* workspace, okc_stream_t stream) {
  if (!workspace) return OKC_ERR_BAD_ARG;
  int32_t* meta = static_cast<int32_t*>(workspace);
  return launch_wait_timeout_probe(meta + kMetaStatus, reinterpret_cast<cudaStream_t>(stream)) == cudaSuccess ? OKC_OK
                                                                                                             : OKC_ERR_CUDA;
}

int okc_moe_read_status(const void* workspace, okc_stream_t stream_, int32_t* detail) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (!workspace) return OKC_ERR_BAD_ARG;
  int32_t host[2] = {0, 0};
  const int32_t* meta = static_cast<const int32_t*>(workspace);
  if (cudaMemcpyAsync(host, meta + kMetaStatus, sizeof(host), cudaMemcpyDeviceToHost, stream) != cudaSuccess) return OKC_ERR_CUDA;
  if (cudaStreamSynchronize(stream) != cudaSuccess) return OKC_ERR_CUDA;
  if (detail) *detail = host[1];
  return host[0];
}

// ---------------------------------------------------------------------------------------------
// Expert-parallel exchange over peer memory.
static bool ep_params(const okc_ep_comm* c, EpParams& p) {
  if (!c || c->world < 1 || c->world > kEpMaxRanks || c->rank < 0 || c->rank >= c->world) return false;
  if (c->tokens <= 0 || (c->tokens % c->world) != 0 || c->hidden <= 0 || (c->hidden % 256) != 0) return false;
  if (c->n_experts <= 0 || (c->n_experts % 4) != 0) return false;
  if (c->wait_limit_ms < 0 || c->reserved[0] != 0 || c->reserved[1] != 0) return false;
  memset(&p, 0, sizeof(p));
  p.wait_ns = c->wait_limit_ms > 0 ? 1000000ull * static_cast<unsigned long long>(c->wait_limit_ms) : 5000000000ull;
  for (int r = 0; r < c->world; ++r) {
    if (!c->peer[r] || !aligned(c->peer[r], 256)) return false;
    p.peer[r] = static_cast<uint8_t*>(c->peer[r]);
  }
  const EpLayout l = ep_layout(c->tokens, c->hidden, c->n_experts);
  p.rank = c->rank; p.world = c->world; p.tokens = c->tokens; p.H = c->hidden; p.E = c->n_experts;
  p.off_hidden = l.off_hidden; p.off_logits = l.off_logits; p.off_partial = l.off_partial;
  return true;
}

uint64_t okc_ep_buffer_bytes(int32_t tokens, int32_t hidden, int32_t n_experts) {
  if (tokens <= 0 || hidden <= 0 || n_experts <= 0) return 0;
  return ep_layout(tokens, hidden, n_experts).total;
}

int okc_ep_views(const okc_ep_comm* comm, void** hidden_all, void** logits_all, void** partial) {
  EpParams p;
  if (!ep_params(comm, p)) return OKC_ERR_BAD_ARG;
  uint8_t* mine = p.peer[p.rank];
  if (hidden_all) *hidden_all = mine + p.off_hidden;
  if (logits_all) *logits_all = mine + p.off_logits;
  if (partial) *partial = mine + p.off_partial;
  return OKC_OK;
}

int okc_ep_gather_tokens(const okc_ep_comm* comm, const void* hidden_own, int64_t hidden_stride,
                         const float* logits_own, okc_stream_t stream) {
  EpParams p;
  if (!ep_params(comm, p)) return OKC_ERR_BAD_ARG;
  if (!hidden_own || !logits_own || !aligned(hidden_own, 16) || !aligned(logits_own, 16)) return OKC_ERR_BAD_ARG;
  if (hidden_stride < p.H || (hidden_stride % 8) != 0) return OKC_ERR_BAD_ARG;
  p.hidden_own = static_cast<const uint16_t*>(hidden_own); p.hidden_stride = hidden_stride; p.logits_own = logits_own;
  return launch_ep_push(p, reinterpret_cast<cudaStream_t>(stream)) == cudaSuccess ? OKC_OK : OKC_ERR_CUDA;
}

int okc_ep_reduce_scatter(const okc_ep_comm* comm, void* out_bf16, okc_stream_t stream) {
  EpParams p;
  if (!ep_params(comm, p)) return OKC_ERR_BAD_ARG;
  if (!out_bf16 || !aligned(out_bf16, 8)) return OKC_ERR_BAD_ARG;
  p.out = static_cast<uint16_t*>(out_bf16);
  return launch_ep_reduce(p, reinterpret_cast<cudaStream_t>(stream)) == cudaSuccess ? OKC_OK : OKC_ERR_CUDA;
}

int okc_ep_routed_views(const okc_ep_comm* comm, int top_k, void** ids_all, void** weights_all) {
  EpParams p;
  if (!ep_params(comm, p) || top_k <= 0 || 2 * top_k > p.E) return OKC_ERR_BAD_ARG;
  uint8_t* mine = p.peer[p.rank];
  if (ids_all) *ids_all = mine + p.off_logits;
  if (weights_all) *weights_all = mine + p.off_logits + static_cast<size_t>(p.tokens) * top_k * 4;
  return OKC_OK;
}

int okc_ep_route_gather(const okc_moe_plan* plan, const okc_ep_comm* comm, const void* hidden_own, int64_t hidden_stride,
                        const float* logits_own, void* workspace, okc_stream_t stream) {
  EpParams p;
  if (!ep_params(comm, p)) return OKC_ERR_BAD_ARG;
  Geometry g;
  if (!plan || !make_geometry(*plan, g)) return OKC_ERR_BAD_PLAN;
  if (plan->n_experts != p.E || plan->hidden != p.H || 2 * plan->top_k > p.E || p.tokens > plan->max_tokens) return OKC_ERR_BAD_PLAN;
  if (!hidden_own || !logits_own || !workspace || !aligned(hidden_own, 16) || !aligned(logits_own, 16) || !aligned(workspace, 256))
    return OKC_ERR_BAD_ARG;
  if (hidden_stride < p.H || (hidden_stride % 8) != 0) return OKC_ERR_BAD_ARG;
  if (!is_sm100()) return OKC_ERR_NO_DEVICE;
  p.hidden_own = static_cast<const uint16_t*>(hidden_own); p.hidden_stride = hidden_stride; p.logits_own = logits_own;
  const int tb = p.tokens / p.world;
  RouteParams rp;
  fill_route_params(plan, g, p.tokens, p.rank * tb, (p.rank + 1) * tb, workspace, rp);
  uint8_t* mine = p.peer[p.rank];
  rp.ids_in = reinterpret_cast<const int32_t*>(mine + p.off_logits);
  rp.wts_in = reinterpret_cast<const float*>(mine + p.off_logits + static_cast<size_t>(p.tokens) * plan->top_k * 4);
  return launch_ep_push_route_sort(p, rp, reinterpret_cast<cudaStream_t>(stream)) == cudaSuccess ? OKC_OK : OKC_ERR_CUDA;
}

int okc_ep_mark_arrived(const okc_ep_comm* comm, int which, int from_rank, okc_stream_t stream) {
  EpParams p;
  if (!ep_params(comm, p)) return OKC_ERR_BAD_ARG;
  if ((which != 0 && which != 1) || from_rank < 0 || from_rank >= p.world) return OKC_ERR_BAD_ARG;
  return launch_ep_mark_arrived(p, which, from_rank, reinterpret_cast<cudaStream_t>(stream)) == cudaSuccess ? OKC_OK
                                                                                                            : OKC_ERR_CUDA;
}

int okc_moe_experts_ep(const okc_moe_plan* plan, const void* packed_w13, const void* packed_w2, const float* gs13,
                       const float* gs2, const void* hidden, int64_t hidden_stride, int T, void* workspace,
                       const okc_ep_comm* comm, void* out_bf16, okc_stream_t stream) {
  EpParams p;
  if (!ep_params(comm, p)) return OKC_ERR_BAD_ARG;
  if (!plan || plan->post_norm != 0) return OKC_ERR_BAD_PLAN;   // the post-expert norm needs whole rows
  if (T != p.tokens || plan->hidden != p.H || !out_bf16 || !aligned(out_bf16, 8)) return OKC_ERR_BAD_ARG;
  p.out = static_cast<uint16_t*>(out_bf16);
  // `out` of the unfused path is not written; the partial sums go to the exchange buffer
  return experts_impl(plan, packed_w13, packed_w2, gs13, gs2, hidden, hidden_stride, T, nullptr, workspace,
                      p.peer[p.rank] + p.off_partial, 1, reinterpret_cast<cudaStream_t>(stream), nullptr, &p);
}

int okc_ep_read_status(const okc_ep_comm* comm, okc_stream_t stream_, int32_t* detail) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  EpParams p;
  if (!ep_params(comm, p)) return OKC_ERR_BAD_ARG;
  int32_t host[2] = {0, 0};
  int32_t* st = reinterpret_cast<int32_t*>(p.peer[p.rank]) + kEpCtrlStatus;
  if (cudaMemcpyAsync(host, st, sizeof(host), cudaMemcpyDeviceToHost, stream) != cudaSuccess) return OKC_ERR_CUDA;
  if (cudaMemsetAsync(st, 0, sizeof(host), stream) != cudaSuccess) return OKC_ERR_CUDA;
  if (cudaStreamSynchronize(stream) != cudaSuccess) return OKC_ERR_CUDA;
  if (detail) *detail = host[1];
  return host[0];
}

// ---------------------------------------------------------------------------------------------
// A step that needs no workspace from the caller.
//
// Some hosts of this library may not allocate device memory at all once they are running: an
// inference server that hands every byte of HBM to its own pool at start-up, a plugin loaded into
// such a server, or code that runs inside a region where cudaMalloc is forbidden or would
// synchronise the device.  For them the step's scratch (the sorted-route tables, the gathered token
// rows, the intermediate activations and the per-route outputs) lives in an array that is part of
// the library image itself.  Every GPU that loads the library carries these 32 MiB until the
// process exits, whether or not this entry point is ever called.
static __device__ __align__(256) unsigned char g_static_scratch[OKC_MOE_STATIC_SCRATCH_BYTES];

// The array's name is only a host-side handle here; the device address has to be asked for, once
// per device, while that device is current.
constexpr int kMaxDevices = 64;
static std::atomic<void*> g_static_scratch_ptr[kMaxDevices];

static int static_scratch_address(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return OKC_ERR_CUDA;
  if (dev < 0 || dev >= kMaxDevices) return OKC_ERR_TOO_LARGE;
  void* p = g_static_scratch_ptr[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr) return OKC_ERR_CUDA;
    g_static_scratch_ptr[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return OKC_OK;
}

int okc_moe_step_static_scratch(const okc_moe_plan* plan, const void* packed_w13, const void* packed_w2,
                                const float* gs13, const float* gs2, const void* hidden, int64_t hidden_stride,
                                const float* logits, int T, int own_t0, int own_t1, const void* post_norm_w,
                                int32_t* ids, float* weights, void* out, int out_f32, okc_stream_t stream) {
  Geometry g;
  if (!plan || !make_geometry(*plan, g)) return OKC_ERR_BAD_PLAN;
  // the plan's workspace (sized by max_tokens) has to fit the array
  if (g.total > static_cast<size_t>(OKC_MOE_STATIC_SCRATCH_BYTES)) return OKC_ERR_TOO_LARGE;
  void* scratch = nullptr;
  const int rc = static_scratch_address(&scratch);
  if (rc != OKC_OK) return rc;
  // The array keeps whatever the previous call left.  Only the control words at its start must
  // read zero before the step; every table behind them is rewritten by the step itself.
  if (cudaMemsetAsync(scratch, 0, kMetaWords * sizeof(int32_t), reinterpret_cast<cudaStream_t>(stream)) != cudaSuccess)
    return OKC_ERR_CUDA;
  return okc_moe_step(plan, packed_w13, packed_w2, gs13, gs2, hidden, hidden_stride, logits, T, own_t0, own_t1,
                      post_norm_w, ids, weights, scratch, out, out_f32, stream);
}

// The status words of the last okc_moe_step_static_scratch on the current device (they live in the
// library's array, out of okc_moe_read_status' reach).  Read them before the next call of that
// entry point: it clears them.
int okc_moe_read_status_static(okc_stream_t stream, int32_t* detail) {
  void* scratch = nullptr;
  const int rc = static_scratch_address(&scratch);
  if (rc != OKC_OK) return rc;
  return okc_moe_read_status(scratch, stream, detail);
}

}  // extern "C"
