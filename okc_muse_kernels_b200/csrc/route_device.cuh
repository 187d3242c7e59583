// Device code of the router shared by the routing kernels (route.cu) and the exchange kernel that routes and
// sorts while it gathers the ranks' tokens (ep.cu): top-k of one token by one warp, token -> expert sort by
// one CTA.
#pragma once
#include "params.cuh"

namespace okc {

// Optional phase clock of the sort (-DOKC_WAIT_PROFILE): thread 0's clock at each phase end.
#ifdef OKC_WAIT_PROFILE
static __device__ long long g_route_prof[8];
#define OKC_ROUTE_MARK(i) { if (threadIdx.x == 0) g_route_prof[i] = clock64(); }
#else
#define OKC_ROUTE_MARK(i)
#endif

constexpr int kRouteThreads = 1024;    // threads of a CTA that sorts a step's routes

__device__ __forceinline__ bool better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }

__device__ __forceinline__ int items_of(int c, bool wide_step, int chunk) {
  const int per = item_rows(c, wide_step, chunk);
  return (c + per - 1) / per;
}

// Top-k of one token by one warp (all 32 lanes call it).  PER = candidates per lane (expert e sits in
// lane e % 32, slot e / 32).  Every lane keeps the best of its untaken candidates; a round is a warp
// arg-max over those 32 values, after which only the winner's lane looks for its next best.  Order:
// larger key first, ties to the lower expert id, NaN never wins.
//   mode 0 (softmax):  key = logit; weights = softmax over the k selected logits.
//   mode 1 (sigmoid):  score = sigmoid(mult * logit), key = score + bias[e]; weights = the selected
//                      scores over (their sum + 1e-15)   (muse_decode_layer/reference.py:419-424,
//                      variants/starter.py:177-182).
// row: the token's E logits, or, with n_part > 1, the first of n_part partial rows part_stride floats
// apart that are added in order.  ids_out / wts_out: the token's k entries.
template <int PER>
__device__ __forceinline__ void topk_token(const float* __restrict__ row, int n_part, size_t part_stride, int E, int k,
                                           int mode, float mult, const float* __restrict__ bias, int lane,
                                           int32_t* __restrict__ ids_out, float* __restrict__ wts_out) {
  float v[PER];    // selection keys
  float sc[PER];   // what the weights are made of (mode 1: the unbiased scores)
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int e = lane + 32 * j;
    float x = -INFINITY;
    if (e < E) {
      x = row[e];
      for (int s = 1; s < n_part; ++s) x += row[static_cast<size_t>(s) * part_stride + e];
    }
    if (mode == 1 && e < E) {
      const float s1 = 1.0f / (1.0f + expf(-x * mult));
      sc[j] = s1;
      x = s1 + (bias != nullptr ? bias[e] : 0.f);
    } else {
      sc[j] = x;
    }
    v[j] = (x == x) ? (x == 0.0f ? 0.0f : x) : -INFINITY;   // NaN never wins; -0 and +0 are one key
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
    // warp arg-max in three warp-wide operations: the largest key (floats mapped to integers of the same order), then
    // the lowest expert id among the lanes that hold it, then that lane's score (expert e sits in lane e % 32)
    const uint32_t bits = __float_as_uint(bv);
    const uint32_t key = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
    const uint32_t kmax = __reduce_max_sync(0xffffffffu, key);
    const int wi = static_cast<int>(__reduce_min_sync(0xffffffffu, key == kmax ? static_cast<uint32_t>(bi) : 0x7fffffffu));
    const float wsc = __shfl_sync(0xffffffffu, bs, wi & 31);
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
    ids_out[lane] = my_id;
    wts_out[lane] = (mode == 1) ? ex / (sum + 1e-15f) : ex / sum;
  }
}

// Token -> expert sort of a step by one CTA of kThreads threads (all of them call it); sm: dynamic
// shared memory of route_smem_bytes(R, slots, kThreads) bytes.  The ids and weights are read past the
// L1 cache (__ldcg): they may have been written by another GPU during this very kernel.
template <int kThreads>
__device__ __forceinline__ void sort_routes_cta(const RouteParams& p, int32_t* sm) {
  const int R = p.T * p.kk;
  // shared memory: rexp int32 [R] (local expert slot or -1) | whist int32 [32][slots] | order int32 [slots]
  // | cnt int32 [slots+1] | offs int32 [slots+1] | ibase int32 [slots+1] | rwt f32 [R]
  int32_t* rexp = sm;
  int32_t* whist = rexp + R;
  int32_t* order = whist + (kThreads / 32) * p.slots;
  int32_t* cnt = order + p.slots;
  int32_t* offs = cnt + p.slots + 1;
  int32_t* ibase = offs + p.slots + 1;
  float* rwt = reinterpret_cast<float*>(ibase + p.slots + 1);     // f32 [R]: the routes' weights
  __shared__ int s_nact;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) s_nact = 0;
  OKC_ROUTE_MARK(0)
  // (asked for here, used by the thread that writes the step's control words at the end: the trip to L2 is over by then)
  int router_gave_up = 0;
  if (tid == 31) router_gave_up = p.meta[kMetaRouterStatus];

  for (int i = tid; i < (kThreads / 32) * p.slots; i += kThreads) whist[i] = 0;
  for (int i = tid; i < R; i += kThreads) p.sorted[i] = -1;

  // ---- 1. the routes' expert slots (global ids outside the local range are skipped)
  for (int i = tid; i < p.T * p.k; i += kThreads) {
    const int t = i / p.k, sl = i - t * p.k;
    const int le = __ldcg(p.ids_in + i) - p.local_start;
    rwt[t * p.kk + sl] = __ldcg(p.wts_in + i);
    rexp[t * p.kk + sl] = (le >= 0 && le < p.local_count) ? le : -1;
  }
  if (p.has_shared)
    for (int t = tid; t < p.T; t += kThreads) {
      rexp[t * p.kk + p.k] = (t >= p.own_t0 && t < p.own_t1) ? p.local_count : -1;
      rwt[t * p.kk + p.k] = 1.0f;
    }
  __syncthreads();
  OKC_ROUTE_MARK(1)

  // ---- 2. per-warp histograms over contiguous chunks of the route list
  const int chunk = ((R + (kThreads / 32) - 1) / (kThreads / 32) + 31) & ~31;
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
  for (int e = tid; e < p.slots; e += kThreads) {
    int run = 0;
    for (int w = 0; w < (kThreads / 32); ++w) {
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
        p.pos[i] = q;
        p.sorted[q] = i;
        p.wsorted[q] = rwt[i];
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
  // (rank of an expert = experts ahead of it; eight neighbouring lanes share one expert's comparisons)
  int active = 0;
  for (int base = 0; base < p.slots; base += kThreads / 8) {
    const int e = base + (tid >> 3), sub = tid & 7;
    const int c = (e < p.slots) ? cnt[e] : 0;
    int rank = 0;
    if (c > 0) {
      for (int o = sub; o < p.slots; o += 8) {
        const int co = cnt[o];
        rank += (co > c || (co == c && o < e)) ? 1 : 0;
      }
    }
    rank += __shfl_xor_sync(0xffffffffu, rank, 1);
    rank += __shfl_xor_sync(0xffffffffu, rank, 2);
    rank += __shfl_xor_sync(0xffffffffu, rank, 4);
    if (c > 0 && sub == 0) {
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
      // a new step: clean status words, unless the router-logits kernel of this very step gave up
      p.meta[kMetaStatus] = router_gave_up ? OKC_ERR_TIMEOUT : 0;
      p.meta[kMetaDetail] = router_gave_up;
      p.meta[kMetaRouterStatus] = 0;
      p.meta[kMetaTokens] = p.T;
      // the widest item is the first one of the heaviest expert
      p.meta[kMetaWcap] = item_pad(min(cmax, item_rows(cmax, wide_step, p.chunk_rows)));
    }
  }
  __syncthreads();
  // the per-call state of the GEMM launch that will work on these routes (the combine kernel behind every GEMM launch
  // clears it too; a step whose predecessor never got that far starts clean all the same)
  for (int i = tid; i < p.max_items; i += kThreads) p.done[i] = 0;
  if (tid < 3) p.meta[kMetaWorkFused + tid] = 0;
  const bool wide_step = s_wide != 0;
  for (int r = tid; r < n_active; r += kThreads) {
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

inline size_t route_smem_bytes(int R, int slots, int threads) {
  return sizeof(int32_t) * (2 * static_cast<size_t>(R) + static_cast<size_t>(threads / 32) * slots + slots + 3 * (slots + 1));
}

}  // namespace okc
