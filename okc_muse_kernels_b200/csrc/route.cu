// Router (softmax top-k: a warp per token over many CTAs) and token -> expert sort (one CTA per step).
//
// Behaviour follows the reference's routing + sort kernels (different algorithm, same results):
//   * top-k with ties to the lowest index       muse_decode_layer/layer.py:394-406 (_routing)
//   * local-expert filter, histogram, offsets   muse_moe_w4a16/submission.py:324-368 (moe_route)
//   * stable (expert, route index) order        muse_moe_w4a16/submission.py:2236-2328 (moe_routegather)
//   * active experts by load, heaviest first    muse_moe_w4a16/submission.py:345-350
// The order inside an expert is deterministic (the reference's moe_route fills it with atomics).
#include <cuda_bf16.h>

#include "route_device.cuh"

namespace okc {



#ifdef OKC_WAIT_PROFILE
extern "C" int okc_moe_debug_route_profile(long long* host_out) {
  return cudaMemcpyFromSymbol(host_out, g_route_prof, sizeof(g_route_prof)) == cudaSuccess ? 0 : -3;
}
#endif

// Router logits from the token rows: part[ks][t][e] = sum over the K range of split ks of
// hidden[t][k] * w[e][k], FP32 multiply-adds in ascending k (bf16 -> f32 is exact).  The step before
// the MoE path in the reference's layer (muse_decode_layer/layer.py:325-351, _router_split), fused
// here with the routing: the logits never exist as a tensor, the top-k kernel adds the splits (in
// split order) as it loads them.  grid (E / 16, splits), 256 threads.
constexpr int kRtE = 16, kRtK = 64, kRtMaxT = 256;
// JT = token groups of 32 the step has (T <= 32 JT): loops over tokens stop there.
template <int JT>
__global__ void __launch_bounds__(256) okc_router_partial(const uint16_t* __restrict__ hidden, int64_t stride,
                                                          const float* __restrict__ w, int T, int H, int E, int kc,
                                                          float* __restrict__ part) {
  __shared__ uint32_t hs[kRtMaxT][kRtK / 2 + 1];   // bf16 pairs, rows padded against bank conflicts
  __shared__ __align__(16) float ws[kRtE][kRtK + 2]; // even row stride: a thread reads k pairs as 8 bytes
  griddep_launch_dependents();   // the top-k kernel may set itself up; it waits for this grid to complete
  // thread = experts e0 + 2 eg, + 1 and tokens tg + 32 j
  const int tid = threadIdx.x, eg = tid & 7, tg = tid >> 3;
  const int e0 = blockIdx.x * kRtE;
  const int k_begin = blockIdx.y * kc, k_end = min(H, k_begin + kc);
  const int n_vec = T * (kRtK / 8);                // 16-byte vectors of the token rows per chunk
  float acc[2][JT];
#pragma unroll
  for (int j = 0; j < JT; ++j) acc[0][j] = acc[1][j] = 0.f;

  // the next chunk travels from global memory into registers while the current one is multiplied
  uint4 hreg[JT];       // 32 JT tokens x 8 vectors / 256 threads
  float4 wreg = make_float4(0.f, 0.f, 0.f, 0.f);
  auto fetch = [&](int k0) {
#pragma unroll
    for (int q = 0; q < JT; ++q) {
      const int i = tid + 256 * q;
      if (i < n_vec) {
        const int t = i >> 3, v = i & 7;
        hreg[q] = *reinterpret_cast<const uint4*>(hidden + static_cast<size_t>(t) * stride + k0 + v * 8);
      }
    }
    wreg = *reinterpret_cast<const float4*>(w + static_cast<size_t>(e0 + (tid >> 4)) * H + k0 + (tid & 15) * 4);
  };
  if (k_begin < k_end) fetch(k_begin);
  for (int k0 = k_begin; k0 < k_end; k0 += kRtK) {
    __syncthreads();                               // the previous chunk has been consumed
#pragma unroll
    for (int q = 0; q < JT; ++q) {
      const int i = tid + 256 * q;
      if (i < n_vec) {
        const int t = i >> 3, v = i & 7;
        hs[t][v * 4 + 0] = hreg[q].x; hs[t][v * 4 + 1] = hreg[q].y; hs[t][v * 4 + 2] = hreg[q].z; hs[t][v * 4 + 3] = hreg[q].w;
      }
    }
    {
      const int r = tid >> 4, v = tid & 15;
      ws[r][v * 4 + 0] = wreg.x; ws[r][v * 4 + 1] = wreg.y; ws[r][v * 4 + 2] = wreg.z; ws[r][v * 4 + 3] = wreg.w;
    }
    __syncthreads();
    if (k0 + kRtK < k_end) fetch(k0 + kRtK);
#pragma unroll 4
    for (int k2 = 0; k2 < kRtK / 2; ++k2) {
      const float2 wa = *reinterpret_cast<const float2*>(&ws[2 * eg][2 * k2]);
      const float2 wb = *reinterpret_cast<const float2*>(&ws[2 * eg + 1][2 * k2]);
#pragma unroll
      for (int j = 0; j < JT; ++j) {
        const int t = tg + 32 * j;
        if (t < T) {
          const uint32_t hv = hs[t][k2];
          const float h0 = __uint_as_float(hv << 16), h1 = __uint_as_float(hv & 0xFFFF0000u);
          acc[0][j] = fmaf(h1, wa.y, fmaf(h0, wa.x, acc[0][j]));
          acc[1][j] = fmaf(h1, wb.y, fmaf(h0, wb.x, acc[1][j]));
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < JT; ++j) {
    const int t = tg + 32 * j;
    if (t < T)
      *reinterpret_cast<float2*>(part + (static_cast<size_t>(blockIdx.y) * T + t) * E + e0 + 2 * eg) =
          make_float2(acc[0][j], acc[1][j]);
  }
}

// Router and sort of a small step in one CTA (T <= 32: a warp per token does the top-k, then all warps
// sort), for logits that are given.  Beyond 32 tokens, or when the logits are split-K partial sums, the top-k of
// all tokens on one SM costs more than spreading them (okc_route_topk_sort_grid).
template <int PER>
__global__ void __launch_bounds__(kRouteThreads, 1) okc_route_topk_sort(const RouteParams p, const float* __restrict__ logits,
                                                                       int n_part) {
  extern __shared__ int32_t sm[];
  griddep_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp < p.T)
    topk_token<PER>(logits + static_cast<size_t>(warp) * p.E, n_part, static_cast<size_t>(p.T) * p.E, p.E, p.k, p.router_mode,
                    p.router_mult, p.router_bias, lane, p.ids_out + warp * p.k, p.wts_out + warp * p.k);
  __threadfence();
  __syncthreads();
  sort_routes_cta<kRouteThreads>(p, sm);
}

// Router and sort of any step in one launch: CTA x does the top-k of tokens [x * per_cta, (x + 1) * per_cta), a warp
// per token, and the CTA that finishes last (a ticket in the control words, which it puts back to zero) sorts the
// whole step.  The tokens spread over the SMs -- what matters when every token's logits are the sum of many
// split-K partial arrays, or when there are hundreds of tokens -- and the sort needs no launch of its own.
template <int PER>
__global__ void __launch_bounds__(kRouteThreads, 1) okc_route_topk_sort_grid(const RouteParams p, const float* __restrict__ logits,
                                                                            int n_part, int per_cta, int stage_parts) {
  extern __shared__ int32_t sm[];
  __shared__ int s_last;
  griddep_wait();
  griddep_launch_dependents();   // the gather kernel may set itself up; it waits for this grid to complete
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (stage_parts) {
    // one token per CTA: all warps fetch the token's partial rows at once, the sums are formed in split order
    float* stage = reinterpret_cast<float*>(sm);     // [n_part][E]
    const int t = blockIdx.x, ev = p.E / 4;
    const float* first = logits + static_cast<size_t>(t) * p.E;
    for (int i = threadIdx.x; i < n_part * ev; i += blockDim.x) {
      const int s = i / ev, c = i - s * ev;
      reinterpret_cast<float4*>(stage)[i] = __ldcg(reinterpret_cast<const float4*>(first + static_cast<size_t>(s) * p.T * p.E) + c);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < p.E; e += blockDim.x) {
      float x = stage[e];
      for (int s = 1; s < n_part; ++s) x += stage[s * p.E + e];
      stage[e] = x;
    }
    __syncthreads();
    if (warp == 0)
      topk_token<PER>(stage, 1, 0, p.E, p.k, p.router_mode, p.router_mult, p.router_bias, lane, p.ids_out + t * p.k,
                      p.wts_out + t * p.k);
  } else {
    const int t = blockIdx.x * per_cta + warp;
    if (warp < per_cta && t < p.T)
      topk_token<PER>(logits + static_cast<size_t>(t) * p.E, n_part, static_cast<size_t>(p.T) * p.E, p.E, p.k, p.router_mode,
                      p.router_mult, p.router_bias, lane, p.ids_out + t * p.k, p.wts_out + t * p.k);
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(&p.meta[kMetaRouteTicket], 1) == static_cast<int>(gridDim.x) - 1) ? 1 : 0;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (threadIdx.x == 0) p.meta[kMetaRouteTicket] = 0;
  sort_routes_cta<kRouteThreads>(p, sm);
}

__global__ void __launch_bounds__(kRouteThreads, 1) okc_route_sort(const RouteParams p) {
  extern __shared__ int32_t sm[];
  griddep_wait();   // the ids may come from the top-k kernel launched just before
  sort_routes_cta<kRouteThreads>(p, sm);
}

// xg[pos] = hidden[token of the route at pos]: rows of the gate_up GEMM's token operand in expert order.
// Block 0 also clears the per-call state of the GEMM launches that follow: their unit counters and
// the per-item completion counts.
__global__ void __launch_bounds__(128) okc_gather_rows(const uint16_t* __restrict__ hidden, int64_t stride,
                                                       int32_t* __restrict__ meta,
                                                       const int32_t* __restrict__ sorted, int kk, int H,
                                                       uint16_t* __restrict__ xg, int32_t* __restrict__ done,
                                                       int max_items) {
  griddep_wait();   // the sort tables come from the kernel before
  griddep_launch_dependents();
  const int q = blockIdx.x;
  if (q == 0) {
    for (int i = threadIdx.x; i < max_items; i += blockDim.x) done[i] = 0;
    if (threadIdx.x < 3) meta[kMetaWorkFused + threadIdx.x] = 0;
  }
  // (the count and the route are requested together, and the row's vectors before the first store: the launch is
  // a chain of dependent trips to L2 otherwise)
  const int n_local = meta[kMetaLocalRoutes];
  const int route = sorted[q];
  if (q >= n_local) return;
  const int t = route / kk;
  const uint4* src = reinterpret_cast<const uint4*>(hidden + static_cast<size_t>(t) * stride);
  uint4* dst = reinterpret_cast<uint4*>(xg + static_cast<size_t>(q) * H);
  const int nvec = H / 8;
  for (int i0 = threadIdx.x; i0 < nvec; i0 += 4 * blockDim.x) {
    uint4 v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (i0 + j * blockDim.x < nvec) v[j] = src[i0 + j * blockDim.x];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (i0 + j * blockDim.x < nvec) dst[i0 + j * blockDim.x] = v[j];
  }
}

// The same gather with the pre-expert RMSNorm of the reference's layer applied on the way
// (muse_decode_layer/layer.py:1700-1745 `moe_gathern`; reference.py:465): the token row, FP32 rows
// rounded to bf16 first, becomes bf16(x * rsqrt(mean(x^2) + eps) * gain[k]).  One CTA per sorted position,
// the row held in registers between the sum of squares and the scaling (H <= 8192).
constexpr int kNormThreads = 256;
constexpr int kNormMaxVec = 4;    // 16-byte vectors of 8 bf16 per thread: H <= 256 * 4 * 8
template <bool F32>
__global__ void __launch_bounds__(kNormThreads) okc_gather_rows_norm(const void* __restrict__ hidden, int64_t stride,
                                                                    const float* __restrict__ gain, float eps,
                                                                    int32_t* __restrict__ meta,
                                                                    const int32_t* __restrict__ sorted, int kk, int H,
                                                                    uint16_t* __restrict__ xg, int32_t* __restrict__ done,
                                                                    int max_items) {
  griddep_wait();
  griddep_launch_dependents();
  const int q = blockIdx.x, tid = threadIdx.x;
  if (q == 0) {
    for (int i = tid; i < max_items; i += blockDim.x) done[i] = 0;
    if (tid < 3) meta[kMetaWorkFused + tid] = 0;
  }
  if (q >= meta[kMetaLocalRoutes]) return;
  const int t = sorted[q] / kk;
  const int nvec = H / 8;
  float v[kNormMaxVec][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kNormMaxVec; ++i) {
    const int o = tid + kNormThreads * i;
    if (o < nvec) {
      if (F32) {
        const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(hidden) + static_cast<size_t>(t) * stride) + 2 * o;
        const float4 a = src[0], b = src[1];
        const float f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] = __bfloat162float(__float2bfloat16_rn(f[j]));
      } else {
        const uint4 u = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(hidden) + static_cast<size_t>(t) * stride)[o];
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          v[i][2 * j] = __uint_as_float(w[j] << 16);
          v[i][2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = fmaf(v[i][j], v[i][j], ss);
    }
  }
  __shared__ float red[kNormThreads / 32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < kNormThreads / 32; ++i) tot += red[i];
  const float r = rsqrtf(tot / static_cast<float>(H) + eps);
  uint4* dst = reinterpret_cast<uint4*>(xg + static_cast<size_t>(q) * H);
#pragma unroll
  for (int i = 0; i < kNormMaxVec; ++i) {
    const int o = tid + kNormThreads * i;
    if (o < nvec) {
      const float4 g0 = reinterpret_cast<const float4*>(gain)[2 * o], g1 = reinterpret_cast<const float4*>(gain)[2 * o + 1];
      const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t lo = __bfloat16_as_ushort(__float2bfloat16_rn(v[i][2 * j] * r * g[2 * j]));
        const uint32_t hi = __bfloat16_as_ushort(__float2bfloat16_rn(v[i][2 * j + 1] * r * g[2 * j + 1]));
        w[j] = lo | (hi << 16);
      }
      dst[o] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

// Exercises the bounded wait on purpose: one warp waits on an mbarrier that nothing ever arrives
// on, with a short limit; the wait gives up and the kernel reports it through the status
// words exactly as the GEMM kernels do (no trap, the context stays usable).
__global__ void okc_wait_timeout_probe(int32_t* status) {
  __shared__ uint64_t bar;
  __shared__ int abort_code;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    abort_code = 0;
    mbar_fence_init();
  }
  __syncthreads();
  const bool ok = mbar_wait(smem_u32(&bar), 0, &abort_code, 0x7e, 1u << 20);
  __syncthreads();
  if (threadIdx.x == 0) {
    status[0] = ok ? OKC_OK : OKC_ERR_TIMEOUT;
    status[1] = abort_code;
  }
}

cudaError_t launch_wait_timeout_probe(int32_t* status, cudaStream_t stream) {
  okc_wait_timeout_probe<<<1, 32, 0, stream>>>(status);
  return cudaGetLastError();
}


cudaError_t launch_route(const RouteParams& p, cudaStream_t stream) {
  const size_t smem = route_smem_bytes(p.T * p.kk, p.slots, kRouteThreads);
  cudaError_t e = cudaFuncSetAttribute(okc_route_sort, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return e;
  if (p.logits != nullptr || p.router_w != nullptr || p.router_w_split != nullptr) {
    // the router proper: ids / weights of every token, then the sort below reads them back
    const float* lg = p.logits;
    int n_part = 0;
    if (p.router_w_split != nullptr) {
      // logits = hidden . router_w^T on the tensor cores (bf16 hi + lo), split-K partial sums in scratch
      n_part = p.router_splits;
      e = launch_router_mma(p.router_wmap, p.router_hmap, p.router_part, p.meta, p.T, p.E, p.H, p.router_kb_per_cta, stream);
      if (e != cudaSuccess) return e;
      lg = p.router_part;
    } else if (p.router_w != nullptr) {
      // logits = hidden . router_w^T as split-K partial sums in scratch; the top-k kernel adds the splits
      n_part = p.router_splits;
      const int kc = ((p.H / kRtK + n_part - 1) / n_part) * kRtK;
      const dim3 rgrid(p.E / kRtE, n_part);
      if (p.T <= 32) okc_router_partial<1><<<rgrid, 256, 0, stream>>>(p.hidden, p.hidden_stride, p.router_w, p.T, p.H, p.E, kc, p.router_part);
      else if (p.T <= 64) okc_router_partial<2><<<rgrid, 256, 0, stream>>>(p.hidden, p.hidden_stride, p.router_w, p.T, p.H, p.E, kc, p.router_part);
      else if (p.T <= 128) okc_router_partial<4><<<rgrid, 256, 0, stream>>>(p.hidden, p.hidden_stride, p.router_w, p.T, p.H, p.E, kc, p.router_part);
      else okc_router_partial<8><<<rgrid, 256, 0, stream>>>(p.hidden, p.hidden_stride, p.router_w, p.T, p.H, p.E, kc, p.router_part);
      e = cudaGetLastError();
      if (e != cudaSuccess) return e;
      lg = p.router_part;
    }
    RouteParams q = p;
    q.logits = nullptr; q.router_w = nullptr; q.router_w_split = nullptr; q.ids_in = p.ids_out; q.wts_in = p.wts_out;
    const dim3 threads(kRouteThreads);
    if (n_part == 0 && p.T <= kRouteThreads / 32) {
      // a small step with its logits given: top-k and sort in one CTA
      const dim3 one(1);
      if (p.E <= 128) {
        e = cudaFuncSetAttribute(okc_route_topk_sort<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        return e != cudaSuccess ? e : launch_kernel(okc_route_topk_sort<4>, one, threads, smem, stream, false, q, lg, n_part);
      }
      if (p.E <= 256) {
        e = cudaFuncSetAttribute(okc_route_topk_sort<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        return e != cudaSuccess ? e : launch_kernel(okc_route_topk_sort<8>, one, threads, smem, stream, false, q, lg, n_part);
      }
      e = cudaFuncSetAttribute(okc_route_topk_sort<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      return e != cudaSuccess ? e : launch_kernel(okc_route_topk_sort<16>, one, threads, smem, stream, false, q, lg, n_part);
    }
    // the tokens over many SMs, the last CTA sorts.  Split-K partial sums: a CTA per token, the partial rows staged
    // in shared memory when they fit.
    const size_t stage_bytes = static_cast<size_t>(n_part) * p.E * sizeof(float);
    const int stage_parts = (n_part > 1 && (p.E % 4) == 0 && stage_bytes <= 160 * 1024) ? 1 : 0;
    const int per_cta = stage_parts ? 1 : (p.T <= 64 ? 4 : 8);
    const size_t smem_g = stage_parts && stage_bytes > smem ? stage_bytes : smem;
    const dim3 grid((p.T + per_cta - 1) / per_cta);
    if (p.E <= 128) {
      e = cudaFuncSetAttribute(okc_route_topk_sort_grid<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_g));
      return e != cudaSuccess ? e : launch_kernel(okc_route_topk_sort_grid<4>, grid, threads, smem_g, stream, n_part > 0, q, lg, n_part, per_cta, stage_parts);
    }
    if (p.E <= 256) {
      e = cudaFuncSetAttribute(okc_route_topk_sort_grid<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_g));
      return e != cudaSuccess ? e : launch_kernel(okc_route_topk_sort_grid<8>, grid, threads, smem_g, stream, n_part > 0, q, lg, n_part, per_cta, stage_parts);
    }
    e = cudaFuncSetAttribute(okc_route_topk_sort_grid<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_g));
    return e != cudaSuccess ? e : launch_kernel(okc_route_topk_sort_grid<16>, grid, threads, smem_g, stream, n_part > 0, q, lg, n_part, per_cta, stage_parts);
  }
  return launch_kernel(okc_route_sort, dim3(1), dim3(kRouteThreads), smem, stream, true, p);
}

cudaError_t launch_gather_norm(const void* hidden, int64_t stride, int hidden_f32, const float* gain, float eps,
                               int32_t* meta, const int32_t* sorted, int kk, int H, int R, void* xg, int32_t* done,
                               int max_items, cudaStream_t stream) {
  if (hidden_f32)
    return launch_kernel(okc_gather_rows_norm<true>, dim3(R), dim3(kNormThreads), 0, stream, true, hidden, stride, gain, eps,
                         meta, sorted, kk, H, static_cast<uint16_t*>(xg), done, max_items);
  return launch_kernel(okc_gather_rows_norm<false>, dim3(R), dim3(kNormThreads), 0, stream, true, hidden, stride, gain, eps,
                       meta, sorted, kk, H, static_cast<uint16_t*>(xg), done, max_items);
}

cudaError_t launch_gather(const void* hidden, int64_t stride, int32_t* meta, const int32_t* sorted, int kk,
                          int H, int R, void* xg, int32_t* done, int max_items, cudaStream_t stream) {
  return launch_kernel(okc_gather_rows, dim3(R), dim3(128), 0, stream, true, static_cast<const uint16_t*>(hidden),
                       stride, meta, sorted, kk, H, static_cast<uint16_t*>(xg), done, max_items);
}

}  // namespace okc
