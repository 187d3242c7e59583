// Router (softmax top-k: a warp per token over many CTAs) and token -> expert sort (one CTA per step).
//
// Behaviour follows the reference's routing + sort kernels (different algorithm, same results):
//   * top-k with ties to the lowest index       muse_decode_layer/layer.py:394-406 (_routing)
//   * local-expert filter, histogram, offsets   muse_moe_w4a16/submission.py:324-368 (moe_route)
//   * stable (expert, route index) order        muse_moe_w4a16/submission.py:2236-2328 (moe_routegather)
//   * active experts by load, heaviest first    muse_moe_w4a16/submission.py:345-350
// The order inside an expert is deterministic (the reference's moe_route fills it with atomics).
#include "params.cuh"

namespace okc {


constexpr int kRouteThreads = 1024;
constexpr int kRouteWarps = kRouteThreads / 32;

// Optional phase clock of the route kernel (-DOKC_WAIT_PROFILE): thread 0's clock at each phase end.
#ifdef OKC_WAIT_PROFILE
__device__ long long g_route_prof[8];
#define OKC_ROUTE_MARK(i) { if (threadIdx.x == 0) g_route_prof[i] = clock64(); }
extern "C" int okc_moe_debug_route_profile(long long* host_out) {
  return cudaMemcpyFromSymbol(host_out, g_route_prof, sizeof(g_route_prof)) == cudaSuccess ? 0 : -3;
}
#else
#define OKC_ROUTE_MARK(i)
#endif

__device__ __forceinline__ bool better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }

__device__ __forceinline__ int items_of(int c, bool wide_step, int chunk) {
  const int per = item_rows(c, wide_step, chunk);
  return (c + per - 1) / per;
}

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

// Top-k of the router, one warp per token, eight tokens per CTA (the tokens of a step spread over
// many SMs: one CTA doing all of them is bound by its own instruction issue).
// PER = candidates per lane (expert e sits in lane e % 32, slot e / 32).  Every lane keeps the best
// of its untaken candidates; a round is a warp arg-max over those 32 values, after which only the
// winner's lane looks for its next best.  Order: larger key first, ties to the lower expert id,
// NaN never wins.
//   mode 0 (softmax):  key = logit; weights = softmax over the k selected logits.
//   mode 1 (sigmoid):  score = sigmoid(mult * logit), key = score + bias[e]; weights = the selected
//                      scores over (their sum + 1e-15)   (muse_decode_layer/reference.py:419-424,
//                      variants/starter.py:177-182).
// The logits are read from `logits` [T, E], or, with n_part > 0, as the sum in split order of the
// n_part arrays [T, E] behind `logits` (the output of okc_router_partial).
template <int PER>
__global__ void __launch_bounds__(256) okc_route_topk(const float* __restrict__ logits, int n_part, int T, int E, int k,
                                                      int mode, float mult, const float* __restrict__ bias,
                                                      int32_t* __restrict__ ids_out, float* __restrict__ wts_out) {
  griddep_wait();                // with n_part > 0 the logits come from the kernel launched just before
  griddep_launch_dependents();   // the sort kernel may set itself up; it waits for this grid to complete
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t >= T) return;
  float v[PER];    // selection keys
  float sc[PER];   // what the weights are made of (mode 1: the unbiased scores)
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int e = lane + 32 * j;
    float x = -INFINITY;
    if (e < E) {
      x = logits[static_cast<size_t>(t) * E + e];
      for (int s = 1; s < n_part; ++s) x += logits[(static_cast<size_t>(s) * T + t) * E + e];
    }
    if (mode == 1 && e < E) {
      const float s1 = 1.0f / (1.0f + expf(-x * mult));
      sc[j] = s1;
      x = s1 + (bias != nullptr ? bias[e] : 0.f);
    } else {
      sc[j] = x;
    }
    v[j] = (x == x) ? x : -INFINITY;
  }
  uint32_t taken = 0;
  float bv = -INFINITY, bs = 0.f;
  int bi = 0x7fffffff;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int e = lane + 32 * j;
    if (e < E && better(v[j], e, bv, bi)) { bv = v[j]; bi = e; bs = sc[j]; }
  }
  float my_val = 0.f;
  int my_id = 0;
  for (int r = 0; r < k; ++r) {
    float wv = bv, wsc = bs;
    int wi = bi;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, wv, o);
      const float os = __shfl_xor_sync(0xffffffffu, wsc, o);
      const int oi = __shfl_xor_sync(0xffffffffu, wi, o);
      if (better(ov, oi, wv, wi)) { wv = ov; wi = oi; wsc = os; }
    }
    if (lane == r) { my_val = wsc; my_id = wi; }
    if (wi == bi) {
      // this lane held the winner: next best of what it has left
      taken |= 1u << (wi >> 5);
      bv = -INFINITY;
      bs = 0.f;
      bi = 0x7fffffff;
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const int e = lane + 32 * j;
        if (e < E && !((taken >> j) & 1u) && better(v[j], e, bv, bi)) { bv = v[j]; bi = e; bs = sc[j]; }
      }
    }
  }
  float ex;
  if (mode == 1) {
    ex = (lane < k) ? my_val : 0.f;
  } else {
    const float top = __shfl_sync(0xffffffffu, my_val, 0);
    ex = (lane < k) ? expf(my_val - top) : 0.f;
  }
  float sum = ex;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (lane < k) {
    ids_out[t * k + lane] = my_id;
    wts_out[t * k + lane] = (mode == 1) ? ex / (sum + 1e-15f) : ex / sum;
  }
}

__global__ void __launch_bounds__(kRouteThreads, 1) okc_route_sort(const RouteParams p) {
  extern __shared__ int32_t sm[];
  const int R = p.T * p.kk;
  // shared memory: rexp int32 [R] (local expert slot or -1) | whist int32 [32][slots] | order int32 [slots]
  // | cnt int32 [slots+1] | offs int32 [slots+1] | ibase int32 [slots+1]
  int32_t* rexp = sm;
  int32_t* whist = rexp + R;
  int32_t* order = whist + kRouteWarps * p.slots;
  int32_t* cnt = order + p.slots;
  int32_t* offs = cnt + p.slots + 1;
  int32_t* ibase = offs + p.slots + 1;
  __shared__ int s_nact;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) s_nact = 0;
  griddep_wait();   // the ids may come from the top-k kernel launched just before
  OKC_ROUTE_MARK(0)

  for (int i = tid; i < kRouteWarps * p.slots; i += kRouteThreads) whist[i] = 0;
  for (int i = tid; i < R; i += kRouteThreads) p.sorted[i] = -1;

  // ---- 1. the routes' expert slots (global ids outside the local range are skipped)
  for (int i = tid; i < p.T * p.k; i += kRouteThreads) {
    const int t = i / p.k, sl = i - t * p.k;
    const int le = p.ids_in[i] - p.local_start;
    rexp[t * p.kk + sl] = (le >= 0 && le < p.local_count) ? le : -1;
  }
  if (p.has_shared)
    for (int t = tid; t < p.T; t += kRouteThreads)
      rexp[t * p.kk + p.k] = (t >= p.own_t0 && t < p.own_t1) ? p.local_count : -1;
  __syncthreads();
  OKC_ROUTE_MARK(1)

  // ---- 2. per-warp histograms over contiguous chunks of the route list
  const int chunk = ((R + kRouteWarps - 1) / kRouteWarps + 31) & ~31;
  const int r0 = warp * chunk;
  for (int b = 0; b < chunk; b += 32) {
    const int i = r0 + b + lane;
    const int e = (i < R) ? rexp[i] : -1;
    const uint32_t m = __match_any_sync(0xffffffffu, e);
    if (e >= 0 && lane == (__ffs(m) - 1)) whist[warp * p.slots + e] += __popc(m);
    __syncwarp();
  }
  __syncthreads();
  // exclusive prefix over warps per expert slot
  for (int e = tid; e < p.slots; e += kRouteThreads) {
    int run = 0;
    for (int w = 0; w < kRouteWarps; ++w) {
      const int c = whist[w * p.slots + e];
      whist[w * p.slots + e] = run;
      run += c;
    }
    cnt[e] = run;
    p.counts[e] = run;
  }
  __syncthreads();
  OKC_ROUTE_MARK(2)
  // ---- 3. offsets (exclusive scan over slots) by warp 0
  if (warp == 0) {
    const int per = (p.slots + 31) >> 5;
    int local = 0;
    for (int j = 0; j < per; ++j) {
      const int e = lane * per + j;
      if (e < p.slots) local += cnt[e];
    }
    int incl = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += n;
    }
    int run = incl - local;
    for (int j = 0; j < per; ++j) {
      const int e = lane * per + j;
      if (e < p.slots) { offs[e] = run; run += cnt[e]; }
    }
    if (lane == 31) { offs[p.slots] = incl; p.counts[p.slots] = incl; }
  }
  __syncthreads();

  OKC_ROUTE_MARK(3)
  // ---- 4. stable positions: offset of the expert + routes of that expert before this one
  for (int b = 0; b < chunk; b += 32) {
    const int i = r0 + b + lane;
    const int e = (i < R) ? rexp[i] : -1;
    const uint32_t m = __match_any_sync(0xffffffffu, e);
    if (i < R) {
      if (e >= 0) {
        const int q = offs[e] + whist[warp * p.slots + e] + __popc(m & ((1u << lane) - 1u));
        const int t = i / p.kk, s = i - t * p.kk;
        float w = 1.0f;
        if (s < p.k) w = p.wts_in[t * p.k + s];
        p.pos[i] = q;
        p.sorted[q] = i;
        p.wsorted[q] = w;
      } else {
        p.pos[i] = -1;
      }
    }
    __syncwarp();
    if (e >= 0 && lane == (31 - __clz(m))) whist[warp * p.slots + e] += __popc(m);
    __syncwarp();
  }

  OKC_ROUTE_MARK(4)
  // ---- 5. work items: experts by load descending (ties by id), cut into runs of item_rows() rows
  int active = 0;
  for (int e = tid; e < p.slots; e += kRouteThreads) {
    const int c = cnt[e];
    if (c > 0) {
      int rank = 0;
      for (int o = 0; o < p.slots; ++o) {
        const int co = cnt[o];
        rank += (co > c || (co == c && o < e)) ? 1 : 0;
      }
      order[rank] = e;
      ++active;
    }
  }
  if (active) atomicAdd(&s_nact, active);
  __syncthreads();
  OKC_ROUTE_MARK(5)
  const int n_active = s_nact;
  __shared__ int s_wide;
  if (warp == 0) {
    const int per = (n_active + 31) >> 5;
    // narrow or wide step: the item counts of both cuts decide (the heaviest expert is order[0])
    int n_narrow = 0, n_wide = 0;
    for (int j = 0; j < per; ++j) {
      const int r = lane * per + j;
      if (r < n_active) {
        n_narrow += items_of(cnt[order[r]], false, p.chunk_rows);
        n_wide += items_of(cnt[order[r]], true, p.chunk_rows);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      n_narrow += __shfl_xor_sync(0xffffffffu, n_narrow, o);
      n_wide += __shfl_xor_sync(0xffffffffu, n_wide, o);
    }
    const int cmax = n_active > 0 ? cnt[order[0]] : 0;
    const bool wide_step = wide_step_pays(cmax, n_narrow, n_wide);
    int local = 0;
    for (int j = 0; j < per; ++j) {
      const int r = lane * per + j;
      if (r < n_active) local += items_of(cnt[order[r]], wide_step, p.chunk_rows);
    }
    int incl = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += n;
    }
    int run = incl - local;
    for (int j = 0; j < per; ++j) {
      const int r = lane * per + j;
      if (r < n_active) { ibase[r] = run; run += items_of(cnt[order[r]], wide_step, p.chunk_rows); }
    }
    if (lane == 31) {
      s_wide = wide_step ? 1 : 0;
      p.meta[kMetaItems] = incl < p.max_items ? incl : p.max_items;
      p.meta[kMetaLocalRoutes] = offs[p.slots];
      p.meta[kMetaStatus] = 0;
      p.meta[kMetaDetail] = 0;
      p.meta[kMetaTokens] = p.T;
      // the widest item is the first one of the heaviest expert
      p.meta[kMetaWcap] = item_pad(min(cmax, item_rows(cmax, wide_step, p.chunk_rows)));
    }
  }
  __syncthreads();
  const bool wide_step = s_wide != 0;
  for (int r = tid; r < n_active; r += kRouteThreads) {
    const int e = order[r];
    const int c = cnt[e];
    int it = ibase[r];
    const int per = item_rows(c, wide_step, p.chunk_rows);
    for (int c0 = 0; c0 < c && it < p.max_items; c0 += per, ++it) {
      const int n = min(per, c - c0);
      p.items[it] = make_int4(e, offs[e] + c0, n, item_pad(n));
    }
  }
  OKC_ROUTE_MARK(6)
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
  if (q >= meta[kMetaLocalRoutes]) return;
  const int t = sorted[q] / kk;
  const uint4* src = reinterpret_cast<const uint4*>(hidden + static_cast<size_t>(t) * stride);
  uint4* dst = reinterpret_cast<uint4*>(xg + static_cast<size_t>(q) * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
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

size_t route_smem_bytes(int R, int slots) {
  return sizeof(int32_t) * (static_cast<size_t>(R) + kRouteWarps * slots + slots + 3 * (slots + 1));
}

cudaError_t launch_route(const RouteParams& p, cudaStream_t stream) {
  const size_t smem = route_smem_bytes(p.T * p.kk, p.slots);
  cudaError_t e = cudaFuncSetAttribute(okc_route_sort, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return e;
  if (p.logits != nullptr || p.router_w != nullptr) {
    // the router proper: ids / weights of every token, then the sort below reads them back
    const float* lg = p.logits;
    int n_part = 0;
    if (p.router_w != nullptr) {
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
    const dim3 grid((p.T + 7) / 8), block(256);
    if (p.E <= 128)
      e = launch_kernel(okc_route_topk<4>, grid, block, 0, stream, n_part > 0, lg, n_part, p.T, p.E, p.k, p.router_mode,
                        p.router_mult, p.router_bias, p.ids_out, p.wts_out);
    else if (p.E <= 256)
      e = launch_kernel(okc_route_topk<8>, grid, block, 0, stream, n_part > 0, lg, n_part, p.T, p.E, p.k, p.router_mode,
                        p.router_mult, p.router_bias, p.ids_out, p.wts_out);
    else
      e = launch_kernel(okc_route_topk<16>, grid, block, 0, stream, n_part > 0, lg, n_part, p.T, p.E, p.k, p.router_mode,
                        p.router_mult, p.router_bias, p.ids_out, p.wts_out);
    if (e != cudaSuccess) return e;
    RouteParams q = p;
    q.logits = nullptr; q.router_w = nullptr; q.ids_in = p.ids_out; q.wts_in = p.wts_out;
    return launch_kernel(okc_route_sort, dim3(1), dim3(kRouteThreads), smem, stream, true, q);
  }
  return launch_kernel(okc_route_sort, dim3(1), dim3(kRouteThreads), smem, stream, true, p);
}

cudaError_t launch_gather(const void* hidden, int64_t stride, int32_t* meta, const int32_t* sorted, int kk,
                          int H, int R, void* xg, int32_t* done, int max_items, cudaStream_t stream) {
  return launch_kernel(okc_gather_rows, dim3(R), dim3(128), 0, stream, true, static_cast<const uint16_t*>(hidden),
                       stride, meta, sorted, kk, H, static_cast<uint16_t*>(xg), done, max_items);
}

}  // namespace okc
