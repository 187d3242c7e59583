// The two exchange steps of the expert-parallel MoE step, written against peer memory: every rank
// maps every other rank's exchange buffer (NVLink / NVSwitch peer access) and the kernels below
// move the data with ordinary stores and loads and order it with system-scope flags.
//
//   push_tokens:  rank r stores its token block (hidden rows, router logits) into every rank's
//                 buffer, then raises flag_in[r] on every rank and waits until all ranks raised
//                 theirs here: an all-gather in one kernel.
//   pull_reduce:  rank r raises flag_rs[r] on every rank ("my partial sums are complete"), waits
//                 for the flags of the others, reads its own token rows of every rank's FP32 partial
//                 sums (rank order, so the sum is deterministic) and writes them as bf16: a
//                 reduce-scatter and the cast in one kernel.
//   combine_reduce: the per-token combine of the local experts' outputs and pull_reduce in one
//                 kernel (the partial sums of a rank's own rows never leave its registers).
//   push_route_sort: push_tokens with the router in it: a rank routes its own tokens (top-k) while it
//                 stores their rows, sends the ids and weights instead of the logits, and the CTA that
//                 has seen every rank's flag sorts the routes of the whole step: three launches and
//                 their gaps fewer on the way to the first GEMM unit.
//
// The reference has no counterpart: its expert all-reduce is not run (muse_moe_w4a16/baseline.py:8).
//
// No buffer is double-buffered and no "done reading" flag exists, because the order of a step
// already protects the data: a rank pushes the tokens of step n+1 only after its pull_reduce of step
// n, which waited for every rank's "partial sums complete" flag of step n, which a rank raises after
// its last read of the step-n tokens; and a rank overwrites its partial sums in step n+1 only after
// its push_tokens of step n+1 saw every rank's step-n+1 flag, which a rank raises after its
// pull_reduce of step n, i.e. after its last read of anybody's step-n partial sums.
//
// Every wait is bounded (five seconds of wall time unless the caller's okc_ep_comm gives a shorter
// limit); a wait that runs out records a code in the buffer's status words and the kernel carries on
// to its end: nothing traps.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/okc_moe.h"
#include "combine_device.cuh"
#include "route_device.cuh"

namespace okc {

namespace {


__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Optional time stamps of a step's exchange kernels (-DOKC_WAIT_PROFILE), in nanoseconds of the GPU's global timer:
// 0 exchange kernel starts (CTA 0, 0), 1 its last CTA has seen all own rows stored and fenced, 2 all ranks' flags seen,
// 3 sort done; 4 combine + reduce kernel starts (CTA 0, 0: the GEMM launch before it is complete), 5 this rank's partial
// sums published, 6 an own-row CTA has seen all ranks' partial sums, 7 the kernel's last CTA leaves.
#ifdef OKC_WAIT_PROFILE
static __device__ unsigned long long g_ep_marks[8];
#define OKC_EP_MARK(i) { if (threadIdx.x == 0) g_ep_marks[i] = global_ns(); }
#else
#define OKC_EP_MARK(i) {}
#endif
__device__ __forceinline__ void st_release_sys(int32_t* p, int32_t v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int32_t ld_acquire_sys(const int32_t* p) {
  int32_t v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_relaxed_sys_f4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// Waits until *flag >= want.  Returns false after limit_ns of wall time.
__device__ __forceinline__ bool wait_flag(const int32_t* flag, int32_t want, unsigned long long limit_ns) {
  if (ld_acquire_sys(flag) >= want) return true;
  const unsigned long long t0 = global_ns();
  for (;;) {
    for (int i = 0; i < 16; ++i) {
      if (ld_acquire_sys(flag) >= want) return true;
      __nanosleep(200);
    }
    if (global_ns() - t0 > limit_ns) return false;
  }
}

__device__ __forceinline__ int32_t* ctrl_of(uint8_t* buf) { return reinterpret_cast<int32_t*>(buf); }
__device__ __forceinline__ int32_t* flags_in_of(uint8_t* buf) { return reinterpret_cast<int32_t*>(buf + kEpOffFlagsIn); }
__device__ __forceinline__ int32_t* flags_rs_of(uint8_t* buf) { return reinterpret_cast<int32_t*>(buf + kEpOffFlagsRs); }

}  // namespace

// grid (row groups, world): CTA (x, r) stores rows x, x + gridDim.x, ... of this rank's block into
// rank r's buffer.  The last CTA to finish signals and waits.
__global__ void __launch_bounds__(256) okc_ep_push_tokens(const EpParams p) {
  uint8_t* mine = p.peer[p.rank];
  uint8_t* dest = p.peer[blockIdx.y];
  const int tb = p.tokens / p.world;
  const int hv = p.H / 8;        // 16-byte vectors per hidden row
  const int lv = p.E / 4;        // 16-byte vectors per logits row
  for (int row = blockIdx.x; row < tb; row += gridDim.x) {
    const uint4* hs = reinterpret_cast<const uint4*>(p.hidden_own + static_cast<size_t>(row) * p.hidden_stride);
    uint4* hd = reinterpret_cast<uint4*>(dest + p.off_hidden) + (static_cast<size_t>(p.rank) * tb + row) * hv;
    for (int i = threadIdx.x; i < hv; i += blockDim.x) hd[i] = hs[i];
    const uint4* ls = reinterpret_cast<const uint4*>(p.logits_own + static_cast<size_t>(row) * p.E);
    uint4* ld = reinterpret_cast<uint4*>(dest + p.off_logits) + (static_cast<size_t>(p.rank) * tb + row) * lv;
    for (int i = threadIdx.x; i < lv; i += blockDim.x) ld[i] = ls[i];
  }
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last;
  int32_t* ctrl = ctrl_of(mine);
  if (threadIdx.x == 0) {
    const int total = gridDim.x * gridDim.y;
    s_last = (atomicAdd(&ctrl[kEpCtrlDoneIn], 1) == total - 1) ? 1 : 0;
  }
  __syncthreads();
  if (!s_last) return;
  // every CTA of this rank has stored (and fenced) its rows: tell everybody, then wait for everybody
  __threadfence_system();
  const int32_t seq = ctrl[kEpCtrlSeqIn] + 1;
  if (threadIdx.x < p.world) {
    st_release_sys(flags_in_of(p.peer[threadIdx.x]) + p.rank, seq);
    if (!wait_flag(flags_in_of(mine) + threadIdx.x, seq, p.wait_ns)) {
      atomicCAS(&ctrl[kEpCtrlStatus], 0, OKC_ERR_TIMEOUT);
      atomicCAS(&ctrl[kEpCtrlDetail], 0, 0x100 | threadIdx.x);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    ctrl[kEpCtrlDoneIn] = 0;
    ctrl[kEpCtrlSeqIn] = seq;
  }
}

// grid (H / 1024, token rows of this rank): thread = four columns of one row.
__global__ void __launch_bounds__(256) okc_ep_pull_reduce(const EpParams p) {
  uint8_t* mine = p.peer[p.rank];
  int32_t* ctrl = ctrl_of(mine);
  const int tb = p.tokens / p.world;
  const int32_t seq = ctrl[kEpCtrlSeqRs] + 1;   // changed only by the last CTA, after every CTA read it
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x < p.world) {
    // this rank's partial sums were written by the kernels before this one in the stream
    __threadfence_system();
    st_release_sys(flags_rs_of(p.peer[threadIdx.x]) + p.rank, seq);
  }
  if (threadIdx.x < p.world) {
    if (!wait_flag(flags_rs_of(mine) + threadIdx.x, seq, p.wait_ns)) {
      atomicCAS(&ctrl[kEpCtrlStatus], 0, OKC_ERR_TIMEOUT);
      atomicCAS(&ctrl[kEpCtrlDetail], 0, 0x200 | threadIdx.x);
    }
  }
  __syncthreads();
  const int row = blockIdx.y;
  const int col = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (col < p.H) {
    const size_t off = (static_cast<size_t>(p.rank) * tb + row) * p.H + col;
    // rank order: the same sum on every run; eight ranks' rows are requested before the first of their adds
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r0 = 0; r0 < p.world; r0 += 8) {
      float4 part[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (r0 + j < p.world) part[j] = ld_relaxed_sys_f4(reinterpret_cast<const float*>(p.peer[r0 + j] + p.off_partial) + off);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (r0 + j < p.world) { acc.x += part[j].x; acc.y += part[j].y; acc.z += part[j].z; acc.w += part[j].w; }
    }
    __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&lo);
    o.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p.out + static_cast<size_t>(row) * p.H + col) = o;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const int total = gridDim.x * gridDim.y;
    if (atomicAdd(&ctrl[kEpCtrlDoneRs], 1) == total - 1) {
      ctrl[kEpCtrlDoneRs] = 0;
      ctrl[kEpCtrlSeqRs] = seq;
    }
  }
}

// The per-token combine of the local experts' outputs and the reduce-scatter in one kernel.
// grid (H / 1024, T); the rows this rank owns are the last block rows.
//   every row t:   acc = sum over the token's local routes (slot order) of y[t * kk + slot]
//   row of a peer: store acc into this rank's partial sums (the owner will load it); the CTA that is
//                  last to publish raises this rank's flag on every rank
//   own row:       wait until every other rank has published its partial sums, add them in rank order
//                  (this rank's acc in its place), round once to bf16
// Only the publishing CTAs are counted towards the flag, and they never wait, so the kernel does not
// need all of its CTAs resident at once: CTAs are handed to the SMs in block order, the publishing
// ones (lower block rows) therefore all run before an own-row CTA can be left waiting for a free SM.
// A second counter over all CTAs tells the one that finishes last to reset both counters and to
// advance the step count (every CTA has read it by then).
__global__ void __launch_bounds__(256) okc_ep_combine_reduce(const EpParams p, const CombineParams c) {
  griddep_wait();    // y comes from the GEMM launch before
  if (blockIdx.x == 0 && blockIdx.y == 0) OKC_EP_MARK(4)
  clear_call_state(c);
  uint8_t* mine = p.peer[p.rank];
  int32_t* ctrl = ctrl_of(mine);
  const int tb = p.tokens / p.world;
  const int own_t0 = p.rank * tb, own_t1 = own_t0 + tb;
  const int32_t seq = ctrl[kEpCtrlSeqRs] + 1;
  int t = static_cast<int>(blockIdx.y) + own_t1;
  if (t >= p.tokens) t -= p.tokens;
  const bool own = t >= own_t0 && t < own_t1;
  const int col = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  const bool live = col < p.H;

  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  if (live) acc = sum_token_routes(c.y, c.pos, t, c.kk, p.H, col);
  if (!own) {
    if (live)
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(mine + p.off_partial) + static_cast<size_t>(t) * p.H + col) = acc;
    // (device scope: the rows are in this GPU's own memory, the CTA that raises the flag fences at system scope)
    __threadfence();
    __syncthreads();
    __shared__ int s_last;
    if (threadIdx.x == 0) {
      const int publishers = gridDim.x * (p.tokens - tb);
      s_last = (atomicAdd(&ctrl[kEpCtrlDoneRs], 1) == publishers - 1) ? 1 : 0;
    }
    __syncthreads();
    if (s_last) {
      // every publishing CTA of this rank has stored (and fenced) its rows
      __threadfence_system();
      if (threadIdx.x < p.world) st_release_sys(flags_rs_of(p.peer[threadIdx.x]) + p.rank, seq);
      OKC_EP_MARK(5)
    }
  } else {
    if (threadIdx.x < p.world && threadIdx.x != p.rank) {
      if (!wait_flag(flags_rs_of(mine) + threadIdx.x, seq, p.wait_ns)) {
        atomicCAS(&ctrl[kEpCtrlStatus], 0, OKC_ERR_TIMEOUT);
        atomicCAS(&ctrl[kEpCtrlDetail], 0, 0x300 | threadIdx.x);
      }
    }
    __syncthreads();
    if (blockIdx.x == 0 && t == own_t0) OKC_EP_MARK(6)
    if (live) {
      const size_t off = static_cast<size_t>(t) * p.H + col;
      // all ranks' rows are requested before the first add (a load per add would put a trip over NVLink between
      // every two adds); the adds run in rank order: the same sum on every run
      float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r0 = 0; r0 < p.world; r0 += 8) {      // eight ranks' rows in flight at a time
        float4 part[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (r0 + j < p.world && r0 + j != p.rank)
            part[j] = ld_relaxed_sys_f4(reinterpret_cast<const float*>(p.peer[r0 + j] + p.off_partial) + off);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (r0 + j < p.world) {
            const float4 v = (r0 + j == p.rank) ? acc : part[j];
            sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
          }
        }
      }
      __nv_bfloat162 lo = __floats2bfloat162_rn(sum.x, sum.y), hi = __floats2bfloat162_rn(sum.z, sum.w);
      uint2 o;
      o.x = *reinterpret_cast<uint32_t*>(&lo);
      o.y = *reinterpret_cast<uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(p.out + static_cast<size_t>(t - own_t0) * p.H + col) = o;
    }
  }
  __syncthreads();   // every thread of the CTA has read the step count
  if (threadIdx.x == 0) {
    const int total = gridDim.x * gridDim.y;
    if (atomicAdd(&ctrl[kEpCtrlDoneAll], 1) == total - 1) {
      OKC_EP_MARK(7)
      ctrl[kEpCtrlDoneRs] = 0;
      ctrl[kEpCtrlDoneAll] = 0;
      ctrl[kEpCtrlSeqRs] = seq;
    }
  }
}

// push_tokens + top-k of the rank's own tokens + the token -> expert sort of the whole step.
// grid (row groups, world), kRouteThreads threads, dynamic shared memory of route_smem_bytes(R, slots, kRouteThreads)
// bytes.
// CTA (x, r): rows x, x + gridDim.x, ... of this rank's block go to rank r's buffer.  The warps of the CTA share the
// routing of those rows (a warp per row: its k ids and weights are stored into the logits area of the buffer, which
// holds ids int32 [T, k], then weights f32 [T, k]), then all warps store the rows themselves.  The last CTA to
// finish raises the flags, waits for every rank's, and sorts with all of its warps.
template <int PER>
__global__ void __launch_bounds__(kRouteThreads, 1) okc_ep_push_route_sort(const EpParams p, const RouteParams rp) {
  extern __shared__ int32_t sm[];
  griddep_wait();
  griddep_launch_dependents();   // the gather kernel may set itself up; it waits for this grid to complete
  if (blockIdx.x == 0 && blockIdx.y == 0) OKC_EP_MARK(0)
  uint8_t* mine = p.peer[p.rank];
  uint8_t* dest = p.peer[blockIdx.y];
  const int tb = p.tokens / p.world;
  const int hv = p.H / 8;        // 16-byte vectors per hidden row
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k = rp.k;
  int32_t* ids_base = reinterpret_cast<int32_t*>(dest + p.off_logits);
  float* wts_base = reinterpret_cast<float*>(dest + p.off_logits + static_cast<size_t>(p.tokens) * k * 4);
  for (int row = blockIdx.x + warp * gridDim.x; row < tb; row += gridDim.x * (kRouteThreads / 32)) {
    const size_t t = static_cast<size_t>(p.rank) * tb + row;
    topk_token<PER>(p.logits_own + static_cast<size_t>(row) * p.E, 1, 0, p.E, k, 0, 1.0f, nullptr, lane, ids_base + t * k,
                    wts_base + t * k);
  }
  for (int row = blockIdx.x; row < tb; row += gridDim.x) {
    const size_t t = static_cast<size_t>(p.rank) * tb + row;
    const uint4* hs = reinterpret_cast<const uint4*>(p.hidden_own + static_cast<size_t>(row) * p.hidden_stride);
    uint4* hd = reinterpret_cast<uint4*>(dest + p.off_hidden) + t * hv;
    for (int i = threadIdx.x; i < hv; i += blockDim.x) hd[i] = hs[i];
  }
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last;
  int32_t* ctrl = ctrl_of(mine);
  if (threadIdx.x == 0) {
    const int total = gridDim.x * gridDim.y;
    s_last = (atomicAdd(&ctrl[kEpCtrlDoneIn], 1) == total - 1) ? 1 : 0;
  }
  __syncthreads();
  if (!s_last) return;
  OKC_EP_MARK(1)
  // every CTA of this rank has stored (and fenced) its rows: tell everybody, then wait for everybody
  __threadfence_system();
  const int32_t seq = ctrl[kEpCtrlSeqIn] + 1;
  if (threadIdx.x < p.world) {
    st_release_sys(flags_in_of(p.peer[threadIdx.x]) + p.rank, seq);
    if (!wait_flag(flags_in_of(mine) + threadIdx.x, seq, p.wait_ns)) {
      atomicCAS(&ctrl[kEpCtrlStatus], 0, OKC_ERR_TIMEOUT);
      atomicCAS(&ctrl[kEpCtrlDetail], 0, 0x100 | threadIdx.x);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    ctrl[kEpCtrlDoneIn] = 0;
    ctrl[kEpCtrlSeqIn] = seq;
  }
  OKC_EP_MARK(2)
  // the ids and weights of all tokens are in this rank's buffer now
  sort_routes_cta<kRouteThreads>(rp, sm);
  __syncthreads();
  OKC_EP_MARK(3)
}

cudaError_t launch_ep_push_route_sort(const EpParams& p, const RouteParams& rp, cudaStream_t stream) {
  const int tb = p.tokens / p.world;
  int gx = 128 / p.world;
  if (gx < 1) gx = 1;
  if (gx > tb) gx = tb;
  const size_t smem = route_smem_bytes(rp.T * rp.kk, rp.slots, kRouteThreads);
  const dim3 grid(gx, p.world), block(kRouteThreads);
  cudaError_t e;
  if (p.E <= 128) {
    e = cudaFuncSetAttribute(okc_ep_push_route_sort<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    return launch_kernel(okc_ep_push_route_sort<4>, grid, block, smem, stream, true, p, rp);
  }
  if (p.E <= 256) {
    e = cudaFuncSetAttribute(okc_ep_push_route_sort<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    return launch_kernel(okc_ep_push_route_sort<8>, grid, block, smem, stream, true, p, rp);
  }
  e = cudaFuncSetAttribute(okc_ep_push_route_sort<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return e;
  return launch_kernel(okc_ep_push_route_sort<16>, grid, block, smem, stream, true, p, rp);
}

// One thread: the flag rank `from` raises on this rank when its part of the coming exchange is in
// place (which = 0 token rows, 1 partial sums), at the value this rank's next wait expects.
__global__ void okc_ep_mark_arrived(const EpParams p, int which, int from) {
  uint8_t* mine = p.peer[p.rank];
  const int32_t* ctrl = ctrl_of(mine);
  if (which == 0) st_release_sys(flags_in_of(mine) + from, ctrl[kEpCtrlSeqIn] + 1);
  else st_release_sys(flags_rs_of(mine) + from, ctrl[kEpCtrlSeqRs] + 1);
}

cudaError_t launch_ep_mark_arrived(const EpParams& p, int which, int from, cudaStream_t stream) {
  okc_ep_mark_arrived<<<1, 1, 0, stream>>>(p, which, from);
  return cudaGetLastError();
}

cudaError_t launch_ep_push(const EpParams& p, cudaStream_t stream) {
  const int tb = p.tokens / p.world;
  int gx = 128 / p.world;
  if (gx < 1) gx = 1;
  if (gx > tb) gx = tb;
  okc_ep_push_tokens<<<dim3(gx, p.world), 256, 0, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_ep_reduce(const EpParams& p, cudaStream_t stream) {
  const int tb = p.tokens / p.world;
  okc_ep_pull_reduce<<<dim3((p.H + 1023) / 1024, tb), 256, 0, stream>>>(p);
  return cudaGetLastError();
}

#ifdef OKC_WAIT_PROFILE
// host_out: unsigned long long [8], the stamps of the last step on the current device
extern "C" int okc_ep_debug_marks(unsigned long long* host_out) {
  return cudaMemcpyFromSymbol(host_out, g_ep_marks, sizeof(g_ep_marks)) == cudaSuccess ? 0 : -3;
}
// host_out: long long [8], the SM clock of thread 0 at the end of each phase of the sort inside the exchange kernel
extern "C" int okc_ep_debug_sort_phases(long long* host_out) {
  return cudaMemcpyFromSymbol(host_out, g_route_prof, sizeof(g_route_prof)) == cudaSuccess ? 0 : -3;
}
#endif

cudaError_t launch_ep_combine_reduce(const EpParams& p, const CombineParams& c, cudaStream_t stream) {
  return launch_kernel(okc_ep_combine_reduce, dim3((p.H + 1023) / 1024, p.tokens), dim3(256), 0, stream, true, p, c);
}

}  // namespace okc
