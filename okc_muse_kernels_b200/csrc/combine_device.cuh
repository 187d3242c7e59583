// The sum over a token's local routes, shared by the combine kernels.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

#include "params.cuh"

namespace okc {

// The combine kernels run behind every GEMM launch; their first CTA puts the per-call state of that launch back to
// zero (its unit counter and the per-item completion counts), so that the next GEMM launch on this workspace needs no
// kernel in front of it to do so.
__device__ __forceinline__ void clear_call_state(const CombineParams& p) {
  if (blockIdx.x == 0 && blockIdx.y == 0) {
    for (int i = threadIdx.x; i < p.max_items; i += blockDim.x) p.done[i] = 0;
    if (threadIdx.x < 3) p.meta[kMetaWorkFused + threadIdx.x] = 0;
  }
}

// acc = sum over slots s = 0 .. kk-1 with pos[t * kk + s] >= 0, in slot order, of the four floats at column `col`
// of y[t * kk + s].  The positions of eight slots and then their rows are all requested before the first add: taken
// one slot at a time, every slot costs two dependent trips to L2 (its position, then its row), which is what a
// small combine launch used to spend most of its time on.  The adds are the same, in the same order.
__device__ __forceinline__ float4 sum_token_routes(const float* __restrict__ y, const int32_t* __restrict__ pos, int t, int kk,
                                                   int H, int col) {
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  const int32_t* ps = pos + t * kk;
  const float* yt = y + static_cast<size_t>(t) * kk * H + col;
  for (int s0 = 0; s0 < kk; s0 += 8) {
    int32_t q[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) q[j] = (s0 + j < kk) ? ps[s0 + j] : -1;
    float4 a[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      a[j] = (q[j] >= 0) ? *reinterpret_cast<const float4*>(yt + static_cast<size_t>(s0 + j) * H) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (q[j] >= 0) { acc.x += a[j].x; acc.y += a[j].y; acc.z += a[j].z; acc.w += a[j].w; }
  }
  return acc;
}

}  // namespace okc
