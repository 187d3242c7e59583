// Kernel parameter blocks and host launchers shared by the translation units of the library.
#pragma once
#include <utility>

#include "format.cuh"

namespace okc {

struct RouteParams {
  const float* logits;
  const int32_t* ids_in;
  const float* wts_in;
  int32_t* ids_out;
  float* wts_out;
  int32_t* meta;
  int32_t* counts;
  int32_t* done;                  // per-item completion counts of the GEMM launch: the sort leaves them (and the unit counters) at zero
  int4* items;
  int32_t* sorted;
  int32_t* pos;
  float* wsorted;
  int T, E, k, kk, slots, local_start, local_count, has_shared, own_t0, own_t1, max_items, chunk_rows;
  // router: 0 = softmax top-k, 1 = sigmoid(mult * logit) + bias chooses, scores renormalised
  int router_mode;
  float router_mult;
  const float* router_bias;       // f32 [E] or null
  // logits from the token rows (null: `logits` is given)
  const float* router_w;          // f32 [E, H]
  const uint16_t* hidden;         // bf16 [T, hidden_stride]
  int64_t hidden_stride;
  int H, router_splits;
  float* router_part;             // scratch f32 [router_splits, T, E]
  // the same logits on the tensor cores: router_w as bf16 hi + lo rows [2 E, H]
  const uint16_t* router_w_split;
  CUtensorMap router_wmap, router_hmap;
  int router_kb_per_cta;
};
cudaError_t launch_router_mma(const CUtensorMap& wmap, const CUtensorMap& hmap, float* part, int32_t* meta, int T, int E, int H,
                              int kb_per_cta, cudaStream_t stream);
cudaError_t launch_router_split(const float* w, void* out, size_t n, cudaStream_t stream);
cudaError_t launch_route(const RouteParams& p, cudaStream_t stream);
cudaError_t launch_gather(const void* hidden, int64_t stride, int32_t* meta, const int32_t* sorted, int kk,
                          int H, int R, void* xg, int32_t* done, int max_items, cudaStream_t stream);

cudaError_t launch_gather_norm(const void* hidden, int64_t stride, int hidden_f32, const float* gain, float eps,
                               int32_t* meta, const int32_t* sorted, int kk, int H, int R, void* xg, int32_t* done,
                               int max_items, cudaStream_t stream);

struct RepackParams {
  const uint8_t* w;
  const uint8_t* sf;
  uint8_t* out;
  int rows, K, pairs, stages, first_slot, count, is_w13, inter;
  size_t expert_bytes;
};
cudaError_t launch_repack(const RepackParams& p, cudaStream_t stream);
struct UnpackParams {
  const uint8_t* packed;
  uint16_t* out;
  int K, pairs, stages, is_w13, inter;
};
cudaError_t launch_unpack(const UnpackParams& p, cudaStream_t stream);

// One of the two GEMM phases of a step: 0 = gate_up on w13 (token operand xg), 1 = down on w2
// (token operand inter).
struct PhaseParams {
  CUtensorMap bmap[5];        // token operand [rows, K] bf16, box = 64 elements x {4, 8, 16, 32, 64} rows
  const uint8_t* wpacked;     // stage images of every expert slot
  const float* gs;            // [slots] global scales
  int pairs;                  // units per work item
  int stages;                 // K / 256
  size_t expert_bytes;
};

// The grouped-GEMM kernel works through the units of phases [phase_lo, phase_hi]: both phases in one
// launch (gate_up units first, then down units, handed out by an atomic counter) or one phase.
struct MoeGemmParams {
  PhaseParams ph[2];
  const int32_t* meta;
  const int4* items;
  int32_t* work_counter;      // units handed out behind the first grid-size ones (zeroed by the combine kernel of the launch before)
  int32_t* done;              // [items] epilogue warps that finished a gate_up unit of the item
  int phase_lo, phase_hi;
  uint16_t* inter;            // bf16 [Rpad, I]     (phase 0 output, phase 1 token operand)
  int I;
  float* y;                   // f32 [R, H]         (phase 1 output)
  const int32_t* sorted;
  const float* wsorted;
  int H;
  int weighted;
  // Token rows of the gate_up phase taken straight from the caller's `hidden` (no gathered copy): one TMA copy
  // per row and 64-element block, the row being the token of the route at that sorted position.
  int direct_rows;
  int kk;                     // routes per token: token of sorted entry s = s / kk
  CUtensorMap hmap;           // hidden [T, H] bf16 with the caller's row stride, box = 64 elements x 1 row
};
cudaError_t launch_gemm(const MoeGemmParams& p, int grid, cudaStream_t stream);

// The exchange kernels of the expert-parallel step (ep.cu).
struct EpParams {
  uint8_t* peer[kEpMaxRanks];   // this process's mapping of every rank's exchange buffer
  int rank, world, tokens, H, E;
  size_t off_hidden, off_logits, off_partial;
  const uint16_t* hidden_own;   // push: bf16 [tokens / world, hidden_stride]
  int64_t hidden_stride;
  const float* logits_own;      // push: f32 [tokens / world, E]
  uint16_t* out;                // reduce: bf16 [tokens / world, H]
  unsigned long long wait_ns;   // limit of every wait on another rank
};
cudaError_t launch_ep_push(const EpParams& p, cudaStream_t stream);
cudaError_t launch_ep_reduce(const EpParams& p, cudaStream_t stream);
cudaError_t launch_ep_push_route_sort(const EpParams& p, const RouteParams& rp, cudaStream_t stream);
cudaError_t launch_ep_mark_arrived(const EpParams& p, int which, int from, cudaStream_t stream);

struct CombineParams {
  const float* y;
  const int32_t* pos;
  const float* wsorted;
  const uint16_t* post_w;
  void* out;
  int kk, H, out_f32;
  int32_t* meta;              // control words and per-item counts of the GEMM launch before: cleared by the first CTA
  int32_t* done;
  int max_items;
};
cudaError_t launch_combine(const CombineParams& p, int T, cudaStream_t stream);
cudaError_t launch_ep_combine_reduce(const EpParams& p, const CombineParams& c, cudaStream_t stream);

cudaError_t launch_cast(const float* in, void* out_bf16, int64_t n, cudaStream_t stream);
cudaError_t launch_wait_timeout_probe(int32_t* status, cudaStream_t stream);

// Launch with (pdl = true) or without the programmatic-serialization attribute.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 bool pdl, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

}  // namespace okc
