// Router logits on the tensor cores: part[split][t][e] = sum over the split's K range of hidden[t][k] * w[e][k],
// with the FP32 router matrix carried as two bf16 matrices, w = hi + lo (hi = bf16(w), lo = bf16(w - hi)), so that
// two bf16 MMAs per K step give the product to about 2^-16 relative -- the reference's way of keeping an FP32
// router on bf16 tensor cores (muse_decode_layer/layer.py:325-351 `_router_split`, pr3_src.cu:28).  The step before
// the MoE path in the reference's layer, fused here with the routing: the logits never exist as a tensor, the top-k
// adds the splits in split order as it loads them.
//
// Swap-AB like the expert GEMMs: the experts fill M (a tile of 128 experts), the tokens are N (T <= 256, padded to
// a multiple of 16), FP32 accumulator in TMEM.  grid (E / 128, splits), 128 threads.  A CTA takes 1..3 K blocks of
// 64 elements: thread 0 starts all their TMA copies at once (hi tile, lo tile, token tile per K block, 128-byte
// swizzle), issues the MMAs as the blocks land (tcgen05.mma, both operands from shared memory), and the four
// warps write the accumulator out as the split's partial sums.  Every wait is bounded.
#include "params.cuh"

namespace okc {

constexpr int kRmTileE = 128;
constexpr int kRmKb = 64;               // K elements per block: one 128-byte swizzled row
constexpr int kRmMaxKb = 3;             // K blocks per CTA (shared memory: 3 x (2 x 16 KB + 32 KB))

// D[tmem] (+)= A[smem] * B[smem]^T
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

struct RouterMmaParams {
  CUtensorMap wmap;        // bf16 [2 E, H]: rows [0, E) hi, [E, 2E) lo; box 64 x 128
  CUtensorMap hmap;        // bf16 [T, stride]: the token rows; box 64 x tpad
  float* part;             // f32 [splits, T, E]
  int32_t* meta;
  int T, E, tpad, kb_per_cta, n_kb, tmem_cols;
};

__global__ void __launch_bounds__(128) okc_router_mma(const __grid_constant__ RouterMmaParams p) {
  extern __shared__ uint8_t smem_raw[];
  griddep_launch_dependents();   // the top-k kernel may set itself up; it waits for this grid to complete
  const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  __shared__ uint64_t bar_full[kRmMaxKb];
  __shared__ uint64_t bar_done;
  __shared__ uint32_t tmem_base;
  __shared__ int abort_code;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int e0 = blockIdx.x * kRmTileE;
  const int kb0 = blockIdx.y * p.kb_per_cta;
  const int nkb = min(p.kb_per_cta, p.n_kb - kb0);
  const uint32_t b_bytes = static_cast<uint32_t>(p.tpad) * 128u;
  const uint32_t blk_bytes = 2u * kRmTileE * 128u + b_bytes;      // hi tile, lo tile, token tile

  if (tid == 0) {
    for (int i = 0; i < kRmMaxKb; ++i) mbar_init(smem_u32(&bar_full[i]), 1);
    mbar_init(smem_u32(&bar_done), 1);
    abort_code = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_base), static_cast<uint32_t>(p.tmem_cols));
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base;

  if (tid == 0 && nkb > 0) {
    tma_prefetch_desc(&p.wmap);
    tma_prefetch_desc(&p.hmap);
    for (int i = 0; i < nkb; ++i) {
      const uint32_t bar = smem_u32(&bar_full[i]);
      const uint32_t dst = smem0 + i * blk_bytes;
      const int k = (kb0 + i) * kRmKb;
      mbar_expect_tx(bar, blk_bytes);
      tma_2d_g2s(dst, &p.wmap, k, e0, bar);
      tma_2d_g2s(dst + kRmTileE * 128, &p.wmap, k, p.E + e0, bar);
      tma_2d_g2s(dst + 2 * kRmTileE * 128, &p.hmap, k, 0, bar);
    }
    const uint32_t idesc = idesc_bf16_m128(static_cast<uint32_t>(p.tpad));
    bool ok = true;
    for (int i = 0; i < nkb && ok; ++i) {
      ok = mbar_wait<100>(smem_u32(&bar_full[i]), 0, &abort_code, 0x51);
      if (!ok) break;
      tc_fence_after();
      const uint32_t a = smem0 + i * blk_bytes;
      const uint64_t a_hi = smem_desc_sw128(a), a_lo = smem_desc_sw128(a + kRmTileE * 128);
      const uint64_t b = smem_desc_sw128(a + 2 * kRmTileE * 128);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {      // K = 16 per MMA: 32 bytes further along the swizzled rows
        mma_ss(tmem, a_hi + 2 * ks, b + 2 * ks, idesc, (i | ks) != 0 ? 1u : 0u);
        mma_ss(tmem, a_lo + 2 * ks, b + 2 * ks, idesc, 1u);
      }
    }
    mma_commit(smem_u32(&bar_done));
    if (!ok) {
      // give the copies a bounded chance to land before the CTA retires
      for (int i = 0; i < nkb; ++i) {
        const long long t0 = clock64();
        while (!mbar_try(smem_u32(&bar_full[i]), 0) && clock64() - t0 < kWaitLimitCycles) {}
      }
    }
  }
  __syncwarp();
  if (nkb > 0) {
    const bool done = mbar_wait<200>(smem_u32(&bar_done), 0, &abort_code, 0x52);
    tc_fence_after();
    if (done && abort_code == 0) {
      // lane = expert row of this warp's 32 TMEM lanes; columns = tokens
      const uint32_t taddr = tmem + (static_cast<uint32_t>(warp * 32) << 16);
      const int e = e0 + warp * 32 + lane;          // (the last tile of an E that is no multiple of 128 has rows beyond E)
      float* dst = p.part + static_cast<size_t>(blockIdx.y) * p.T * p.E + e;
      for (int c0 = 0; c0 < p.tpad; c0 += 16) {
        uint32_t r[16];
        tmem_ld16(taddr + c0, r);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (c0 + j < p.T && e < p.E) dst[static_cast<size_t>(c0 + j) * p.E] = __uint_as_float(r[j]);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, static_cast<uint32_t>(p.tmem_cols));
  }
  if (tid == 0 && abort_code != 0) {
    // the sort kernel of the same step takes this over into the step's status words
    atomicCAS(&p.meta[kMetaRouterStatus], 0, 0x500 | abort_code);
  }
}

// w f32 [E, H] -> bf16 [2 E, H]: rows [0, E) = bf16(w), rows [E, 2 E) = bf16(w - bf16(w)).
__global__ void __launch_bounds__(256) okc_router_split(const float* __restrict__ w, uint16_t* __restrict__ out, size_t n) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float x = w[i];
  const uint32_t xb = __float_as_uint(x);
  // round to nearest even to bf16, by hand (no header types needed)
  const uint32_t hi_bits = (xb + 0x7FFFu + ((xb >> 16) & 1u)) & 0xFFFF0000u;
  const float hi = (x == x) ? __uint_as_float(hi_bits) : x;
  const float rest = x - hi;
  const uint32_t rb = __float_as_uint(rest);
  const uint32_t lo_bits = (rb + 0x7FFFu + ((rb >> 16) & 1u)) >> 16;
  out[i] = static_cast<uint16_t>(__float_as_uint(hi) >> 16);
  out[n + i] = static_cast<uint16_t>(lo_bits);
}

cudaError_t launch_router_split(const float* w, void* out, size_t n, cudaStream_t stream) {
  okc_router_split<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(w, static_cast<uint16_t*>(out), n);
  return cudaGetLastError();
}

size_t router_mma_smem_bytes(int kb_per_cta, int tpad) {
  return 1024 + static_cast<size_t>(kb_per_cta) * (2 * kRmTileE * 128 + static_cast<size_t>(tpad) * 128);
}

// kb_per_cta K blocks per CTA, splits = ceil(H / 64 / kb_per_cta) partial sums [T, E] behind `part`.
cudaError_t launch_router_mma(const CUtensorMap& wmap, const CUtensorMap& hmap, float* part, int32_t* meta, int T, int E, int H,
                              int kb_per_cta, cudaStream_t stream) {
  RouterMmaParams p;
  p.wmap = wmap; p.hmap = hmap; p.part = part; p.meta = meta; p.T = T; p.E = E;
  p.tpad = (T + 15) & ~15;
  p.kb_per_cta = kb_per_cta;
  p.n_kb = H / kRmKb;
  p.tmem_cols = p.tpad <= 32 ? 32 : p.tpad <= 64 ? 64 : p.tpad <= 128 ? 128 : 256;
  const int splits = (p.n_kb + kb_per_cta - 1) / kb_per_cta;
  const size_t smem = router_mma_smem_bytes(kb_per_cta, p.tpad);
  cudaError_t e = cudaFuncSetAttribute(okc_router_mma, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return e;
  okc_router_mma<<<dim3((E + kRmTileE - 1) / kRmTileE, splits), 128, smem, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace okc
